"""Next-token choice.  Greedy when temperature <= 0, else temperature sampling by
inverse CDF (crates/bitnet-core/src/llama/runtime.rs:81-107); the reference has no
other sampling option (no top-k, top-p or penalties), and neither has this
library.  The choice itself is a CUDA kernel (``CudaOps.sample``)."""
from .rng import uniform, uniforms

__all__ = ["uniform", "uniforms"]
