"""Host-side binding of libtei_b200.so: the `Backend` mirror (`backend`), the kernel-level
wrappers used by tests and the benchmark (`ops`), the batching queue (`queue`) and the ctypes
loader (`_lib`)."""
from .backend import B200Backend, BackendError, Batch, Embedding, plan_shards  # noqa: F401
from .queue import BatchQueue  # noqa: F401,E402
