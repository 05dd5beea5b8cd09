"""ojas-cuda for B200: the nanolab GPT training step behind ojas's Backend operator API.

The compute is hand-written sm_100a CUDA in libojas_cuda.so (C ABI: include/ojas_cuda.h); this
package is the host-side mirror of the reference interface used by the tests and the bench.
"""
from .backend import (CudaBackend, DType, OjasError, Tensor, Trainer, TrainConfig, ModelSpec, AdamWConfig, MuonNs5Config, Session,  # noqa: F401
                      STATUS_NAMES)
