"""Host-side checks that run without a GPU: token id validation and padding trim of get_rows, shape checks of
add_row_bias — the errors the reference raises before it touches the device
(src/ggml/hip_backend/ops/get_rows.rs:84-94, src/backend/hip_backend/backend.rs:924-946)."""
import numpy as np
import pytest

from rocmforge_b200 import ops, projections


def test_validate_token_ids_names_the_first_bad_id():
    ops.validate_token_ids([0, 5, 99], 100)
    ops.validate_token_ids([], 1)
    with pytest.raises(ValueError, match="Token ID 100 exceeds vocab size 100"):
        ops.validate_token_ids([3, 100, 200], 100)


def test_get_rows_validates_before_touching_the_backend():
    class NoBackend:          # any use of the library would raise AttributeError instead of ValueError
        pass
    with pytest.raises(ValueError, match="Token ID 7 exceeds vocab size 7"):
        ops.get_rows(NoBackend(), object(), np.array([1, 7], dtype=np.uint32), 64, 7, object())
    # trailing padding is dropped first, so a bad id behind the first 0 is never seen (execute_get_rows' order)
    with pytest.raises(AttributeError):
        ops.get_rows(NoBackend(), b"", np.array([1, 0, 9], dtype=np.uint32), 64, 7, object(), qtype=0, trim_padding=True)


def test_add_row_bias_shape_errors_and_empty_tensor():
    class NoBackend:
        pass
    with pytest.raises(ValueError, match="Tensor for row bias must be 2D"):
        projections.add_row_bias(NoBackend(), object(), (4, 5, 6), object(), (6,))
    with pytest.raises(ValueError, match=r"Bias shape \[2, 6\] incompatible with tensor shape \[4, 6\]"):
        projections.add_row_bias(NoBackend(), object(), (4, 6), object(), (2, 6))
    projections.add_row_bias(NoBackend(), object(), (0, 6), object(), (6,))       # rows == 0: nothing to do
    projections.add_row_bias(NoBackend(), object(), (4, 0), object(), (1, 0))     # cols == 0: nothing to do
