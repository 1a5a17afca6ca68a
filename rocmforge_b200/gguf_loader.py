"""Host mirror of the reference's GGUF loader for the quantized-weight path.

GgufLoader / GgufMetadata / LazyTensor keep the names and field meaning of src/loader/gguf/types.rs,
src/loader/metadata.rs and src/loader/lazy_tensor.rs:49-75; parsing and mapping are done by the C
library (b200q_gguf_*). load_tensor_to_gpu hands out packed device tensors (QuantizedWeight) cached by
name, where the reference dequantises to fp32 (src/loader/gguf/types.rs:199-254).
"""
import ctypes
from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

import numpy as np

from . import _lib
from ._lib import check
from .backend import QuantizedWeight

# GgufTensorType ids -> names (src/loader/tensor_type.rs:63-78); 39 is ggml's own MXFP4 id
TYPE_NAMES = {0: "FP32", 1: "FP16", 2: "Q4_0", 8: "Q8_0", 10: "Q2_K", 11: "Q3_K", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K",
              20: "MXFP4", 21: "MXFP6_E2M3", 22: "MXFP6_E3M2", 39: "MXFP4"}


@dataclass
class LazyTensor:
    """Metadata-only handle; the bytes stay in the mapped file until they are asked for."""
    name: str
    offset: int
    size: int
    shape: Tuple[int, ...]
    tensor_type: str
    index: int
    qtype: int
    n: int
    k: int


@dataclass
class GgufMetadata:
    """Hyper-parameters the reference collects while parsing (update_metadata, src/loader/gguf/metadata.rs:271-369)."""
    architecture: str = ""
    file_type: int = 0
    num_layers: int = 0
    num_heads: int = 0
    num_kv_heads: Optional[int] = None
    hidden_size: int = 0
    intermediate_size: int = 0
    head_dim: int = 0
    max_position_embeddings: int = 2048
    vocab_size: int = 0
    rms_norm_eps: float = 1e-6
    embedded_tokenizer_json: Optional[str] = None
    raw: Dict[str, str] = field(default_factory=dict)


def _int(v, default=0):
    try:
        return int(v)
    except ValueError:
        return default


def _float(v, default):
    try:
        return float(v)
    except ValueError:
        return default


# key -> (field, kind) exactly as the reference's table reads them (src/loader/gguf/metadata.rs:271-369)
_INT_KEYS = {
    "general.file_type": "file_type",
    "glm.n_layers": "num_layers", "glm.n_heads": "num_heads", "glm.n_embd": "hidden_size",
    "glm.intermediate_size": "intermediate_size", "glm.head_dim": "head_dim", "glm.vocab_size": "vocab_size",
    "gemma3.embedding_length": "hidden_size", "gemma3.block_count": "num_layers",
    "gemma3.feed_forward_length": "intermediate_size", "gemma3.attention.head_count": "num_heads",
    "gemma3.attention.head_count_kv": "num_kv_heads", "gemma3.attention.key_length": "head_dim",
    "gemma3.attention.value_length": "head_dim",
    "qwen2.block_count": "num_layers", "qwen2.attention.head_count": "num_heads",
    "qwen2.attention.head_count_kv": "num_kv_heads", "qwen2.embedding_length": "hidden_size",
    "qwen2.intermediate_size": "intermediate_size", "qwen2.vocab_size": "vocab_size",
    "llama.block_count": "num_layers", "llama.attention.head_count": "num_heads",
    "llama.attention.head_count_kv": "num_kv_heads", "llama.embedding_length": "hidden_size",
    "llama.feed_forward_length": "intermediate_size", "llama.vocab_size": "vocab_size",
}
_CTX_KEYS = ("glm.max_position_embeddings", "gemma3.context_length", "qwen2.max_position_embeddings",
             "llama.max_position_embeddings")
_EPS_KEYS = ("glm.rms_norm_eps", "gemma3.attention.layer_norm_rms_epsilon", "llama.attention.layer_norm_rms_epsilon",
             "qwen2.attention.layer_norm_rms_epsilon", "qwen2.attention_norm_epsilon")
_ROPE_KEYS = ("qwen2.rope.dimension_count", "llama.rope.dimension_count")


def update_metadata(md: GgufMetadata, key: str, value: str) -> None:
    """One key/value pair -> metadata fields; same keys, same defaults when a value does not parse."""
    if key == "general.architecture":
        md.architecture = value
    elif key in _INT_KEYS:
        setattr(md, _INT_KEYS[key], _int(value))
    elif key in _CTX_KEYS:
        md.max_position_embeddings = _int(value, 2048)
    elif key in _EPS_KEYS:
        md.rms_norm_eps = _float(value, 1e-6)
    elif key in _ROPE_KEYS:
        if _int(value) > 0:          # a zero or unparsable rope dimension leaves head_dim alone
            md.head_dim = _int(value)
    elif key == "tokenizer.json" or key.endswith(".tokenizer_json"):
        if md.embedded_tokenizer_json is None:
            md.embedded_tokenizer_json = value


def layer_tensor_names(layer: int) -> Dict[str, str]:
    """GGUF tensor names of one transformer block's projections
    (src/model/execution_plan/layer_tensors.rs:28-101): fused attn_qkv or separate attn_q/k/v, attn_output,
    ffn_gate / ffn_up / ffn_down."""
    p = f"blk.{layer}"
    return {"attn_qkv": f"{p}.attn_qkv.weight", "attn_q": f"{p}.attn_q.weight", "attn_k": f"{p}.attn_k.weight",
            "attn_v": f"{p}.attn_v.weight", "attn_output": f"{p}.attn_output.weight",
            "ffn_gate": f"{p}.ffn_gate.weight", "ffn_up": f"{p}.ffn_up.weight", "ffn_down": f"{p}.ffn_down.weight"}


class GgufLoader:
    """Opens a GGUF file, exposes its metadata and lazy tensor handles, uploads packed tensors on demand."""

    def __init__(self, path, reference_fixture=False):
        self.lib = _lib.load()
        self.path = str(path)
        h = ctypes.c_void_p()
        check(self.lib.b200q_gguf_open(self.path.encode(), _lib.GGUF_REFERENCE_FIXTURE if reference_fixture else 0,
                                       ctypes.byref(h)))
        self.handle = h
        self.metadata = GgufMetadata()
        for i in range(self.lib.b200q_gguf_kv_count(h)):
            key, vt = ctypes.c_char_p(), ctypes.c_int()
            check(self.lib.b200q_gguf_kv_key(h, i, ctypes.byref(key), ctypes.byref(vt)))
            need = ctypes.c_size_t()
            check(self.lib.b200q_gguf_meta_string(h, key.value, None, 0, ctypes.byref(need)))
            buf = ctypes.create_string_buffer(need.value)
            check(self.lib.b200q_gguf_meta_string(h, key.value, buf, need.value, None))
            k, v = key.value.decode("utf-8", "replace"), buf.value.decode("utf-8", "replace")
            self.metadata.raw[k] = v
            update_metadata(self.metadata, k, v)
        self.lazy_tensors: Dict[str, LazyTensor] = {}
        for i in range(self.lib.b200q_gguf_tensor_count(h)):
            t = _lib.GgufTensorInfo()
            check(self.lib.b200q_gguf_tensor_info(h, i, ctypes.byref(t)))
            name = t.name.decode("utf-8", "replace")
            self.lazy_tensors[name] = LazyTensor(name, t.file_offset, t.nbytes, tuple(t.dims[:t.n_dims]),
                                                 TYPE_NAMES.get(t.ggml_type, str(t.ggml_type)), i, t.qtype, t.n, t.k)
        self.gpu_cache: Dict[Tuple[str, int, int], QuantizedWeight] = {}
        self.arenas = []

    def tensor_names(self):
        return list(self.lazy_tensors)

    def tensor_bytes(self, name) -> np.ndarray:
        """The mapped bytes of a tensor (read-only view; valid until close)."""
        lt = self.lazy_tensors[name]
        p, n = ctypes.c_void_p(), ctypes.c_size_t()
        check(self.lib.b200q_gguf_tensor_data(self.handle, lt.index, ctypes.byref(p), ctypes.byref(n)))
        if n.value == 0:
            return np.empty(0, dtype=np.uint8)
        buf = (ctypes.c_uint8 * n.value).from_address(p.value)
        a = np.frombuffer(buf, dtype=np.uint8)
        a.flags.writeable = False
        return a

    def load_tensor_to_gpu(self, name, backend, shard_rank=0, shard_count=1) -> QuantizedWeight:
        """Upload once, then serve from the cache, like the reference's gpu_cache keyed by tensor name."""
        key = (name, shard_rank, shard_count)
        if key in self.gpu_cache:
            return self.gpu_cache[key]
        if name not in self.lazy_tensors:
            raise KeyError(f"Tensor '{name}' not found")
        h = ctypes.c_void_p()
        check(self.lib.b200q_gguf_upload_tensor(backend.ctx, self.handle, self.lazy_tensors[name].index, shard_rank,
                                                shard_count, ctypes.byref(h)))
        w = QuantizedWeight.from_handle(backend, h)
        self.gpu_cache[key] = w
        return w

    def load_to_gpu(self, backend, names=None, shard_rank=0, shard_count=1) -> Dict[str, QuantizedWeight]:
        """Every quantized tensor this library has a kernel for (or the ones named), uploaded."""
        out = {}
        for name, lt in self.lazy_tensors.items():
            if names is not None and name not in names:
                continue
            if lt.qtype < 0:
                continue
            out[name] = self.load_tensor_to_gpu(name, backend, shard_rank, shard_count)
        return out

    def load_to_gpu_async(self, backend, shard_rank=0, shard_count=1) -> Dict[str, QuantizedWeight]:
        """GgufLoader::load_to_gpu_async (src/loader/gguf/types.rs:326): every tensor with packed kernels goes into ONE
        arena sized for exactly them (arena_upload_phase, gpu_upload.rs:413-594); copies and layout kernels are queued
        on the backend's stream and this returns without waiting for them. The weights enter the cache under their
        names, so load_tensor_to_gpu serves them afterwards."""
        from .backend import WeightArena
        n = len(self.lazy_tensors)
        handles = (ctypes.c_void_p * n)()
        arena = ctypes.c_void_p()
        check(self.lib.b200q_gguf_upload_all(backend.ctx, self.handle, shard_rank, shard_count, ctypes.byref(arena), handles, n))
        self.arenas.append(WeightArena(backend, handle=arena))
        out = {}
        for name, lt in self.lazy_tensors.items():
            h = handles[lt.index]
            if not h:
                continue
            w = QuantizedWeight.from_handle(backend, ctypes.c_void_p(h))
            old = self.gpu_cache.pop((name, shard_rank, shard_count), None)
            if old is not None:
                old.free()
            self.gpu_cache[(name, shard_rank, shard_count)] = w
            out[name] = w
        return out

    def close(self):
        for w in self.gpu_cache.values():
            w.free()
        self.gpu_cache.clear()
        for a in getattr(self, "arenas", []):
            a.free()
        self.arenas = []
        if self.handle:
            self.lib.b200q_gguf_close(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
