"""checkers_b200 -- B200 (sm_100a) implementation of the Checkers
checkpoint-compression path: tensor statistics and clustering, the low-byte
split, byte histograms, 256-lane rANS encode/decode and the reference's
.ansc/.mant/.dict files.  All compute runs in libcheckers_b200.so; importing
this package fails if that library has not been built."""
from . import _lib
from ._lib import (BF16, CAT_EXP_AVG, CAT_EXP_AVG_SQ, CAT_MASTER, CAT_MODEL, DTYPE_UNKNOWN, ELEM_SIZE, F16, F32, I8,
                   I32, CheckersError)
from .api import (analyze_tensors, compress_and_save, current_context, initialize_context, load_and_decompress,
                  register_tensors)
from .context import STATIC_MAX_TENSOR_BYTES, Context, encode_tensor_static, normalize_histogram
from .manifest import build_manifest, gather_summaries, write_manifest

__all__ = ["Context", "CheckersError", "initialize_context", "analyze_tensors", "compress_and_save",
           "load_and_decompress", "register_tensors", "current_context", "normalize_histogram", "build_manifest",
           "gather_summaries", "write_manifest", "encode_tensor_static", "STATIC_MAX_TENSOR_BYTES", "F32", "BF16", "F16", "I8", "I32"]
