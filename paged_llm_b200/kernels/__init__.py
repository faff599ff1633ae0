"""Python side of the CUDA kernels: `ops.CudaOps` (the library the parts call)
and `plan` (host-side work lists for attention)."""
