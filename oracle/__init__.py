"""CPU oracle for the quantized-weight matmul path -- test infrastructure only.

Only tests, the smoke check and the benchmark's CPU-baseline legs may import this
package; the shipped library never does.
"""
