"""sfnx_b200: B200 (sm_100a) kernels of the speculative-decoding verify window behind a C ABI (include/sfnx_b200.h)."""
from . import lib  # noqa: F401
