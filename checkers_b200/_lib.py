"""ctypes binding of libcheckers_b200.so (the C ABI in include/checkers_b200.h).

There is no CPU implementation behind this module: if the CUDA library is
missing or cannot be loaded, importing it raises."""
import ctypes as C
import os

from .build import LIB

CHK_OK = 0
F32, BF16, F16, I8, I32, DTYPE_UNKNOWN = 0, 1, 2, 3, 4, 255
CAT_MODEL, CAT_MASTER, CAT_EXP_AVG, CAT_EXP_AVG_SQ, CAT_UNKNOWN = 0, 1, 2, 3, 255
ELEM_SIZE = {F32: 4, BF16: 2, F16: 2, I8: 1, I32: 4}


class Summary(C.Structure):
    _fields_ = [("n_tensors", C.c_uint64), ("n_tables", C.c_uint64), ("states_bytes", C.c_uint64),
                ("mantissa_bytes", C.c_uint64), ("dict_bytes", C.c_uint64), ("original_bytes", C.c_uint64)]


class CheckersError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"[checkers_b200] error {code}: {message}")
        self.code = code


def _load():
    if not os.path.exists(LIB):
        raise ImportError(f"{LIB} is missing: build it with `python -m checkers_b200.build` "
                          "(nvcc, sm_100a). There is no CPU fallback.")
    lib = C.CDLL(LIB)
    vp, u64, u32p, f32p = C.c_void_p, C.c_uint64, C.POINTER(C.c_uint32), C.POINTER(C.c_float)
    sig = {
        "chk_last_error": (C.c_char_p, []),
        "chk_context_create": (C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(vp)]),
        "chk_context_create_ex": (C.c_int, [C.c_int, C.c_int, C.c_int, u64, C.POINTER(vp)]),
        "chk_context_destroy": (C.c_int, [vp]),
        "chk_reset": (C.c_int, [vp]),
        "chk_release_workspace": (C.c_int, [vp]),
        "chk_set_histogram_bins": (C.c_int, [vp, C.c_uint32]),
        "chk_register_tensor": (C.c_int, [vp, C.c_char_p, vp, u64, C.c_uint8, C.c_uint8]),
        "chk_tensor_count": (C.c_int, [vp, C.POINTER(u64)]),
        "chk_set_option": (C.c_int, [vp, C.c_char_p, C.c_int64]),
        "chk_analyze": (C.c_int, [vp]),
        "chk_shared_model_cost": (C.c_int, [vp, C.POINTER(u64), u64, C.POINTER(C.c_double), C.POINTER(u64)]),
        "chk_hll_sketch_all": (C.c_int, [vp]),
        "chk_hll_get": (C.c_int, [vp, u64, C.POINTER(C.c_uint8)]),
        "chk_hll_merge": (C.c_int, [C.POINTER(C.c_uint8), C.POINTER(C.c_uint8)]),
        "chk_hll_count": (C.c_int, [C.POINTER(C.c_uint8), C.POINTER(C.c_double)]),
        "chk_shared_vocabulary_report": (C.c_int, [vp, C.POINTER(u64), C.POINTER(u64)]),
        "chk_get_tensor_stats": (C.c_int, [vp, u64, u32p, f32p, f32p, f32p]),
        "chk_get_cluster_ids": (C.c_int, [vp, C.POINTER(C.c_int32), u64, C.POINTER(C.c_int32)]),
        "chk_get_cluster_anchor": (C.c_int, [vp, C.c_int32, C.c_char_p]),
        "chk_set_cluster_info": (C.c_int, [vp, u64, C.POINTER(C.c_char_p), C.POINTER(C.c_int32), C.c_int32,
                                           C.POINTER(C.c_char_p)]),
        "chk_compress_and_save": (C.c_int, [vp, C.c_char_p]),
        "chk_compress": (C.c_int, [vp, C.c_int]),
        "chk_get_image": (C.c_int, [vp, C.c_int, C.POINTER(vp), C.POINTER(u64)]),
        "chk_get_summary": (C.c_int, [vp, C.POINTER(Summary)]),
        "chk_get_table_report": (C.c_int, [vp, C.POINTER(u64), C.POINTER(u64)]),
        "chk_load_and_decompress": (C.c_int, [vp, C.c_char_p]),
        "chk_decompress_images": (C.c_int, [vp, vp, u64, vp, u64, vp, u64]),
        "chk_decompress_resident": (C.c_int, [vp, C.POINTER(vp)]),
        "chk_restored_count": (C.c_int, [vp, C.POINTER(u64)]),
        "chk_split": (C.c_int, [vp, vp, u64, C.c_uint8, vp, vp]),
        "chk_merge": (C.c_int, [vp, vp, vp, u64, C.c_uint8, vp]),
        "chk_byte_histogram": (C.c_int, [vp, vp, u64, u32p]),
        "chk_normalize_histogram": (C.c_int, [u32p, C.c_int, C.c_int, u32p, u32p, u32p, u32p]),
        "chk_get_timing": (C.c_int, [vp, C.c_char_p, C.POINTER(C.c_double)]),
        "chk_kernel_launches": (C.c_int, [vp, C.POINTER(u64)]),
        "chk_get_stream": (C.c_int, [vp, C.POINTER(vp)]),
        "chk_stream_create": (C.c_int, [C.c_int, C.c_int, u64, C.c_int, C.POINTER(vp)]),
        "chk_stream_set_option": (C.c_int, [vp, C.c_char_p, C.c_int64]),
        "chk_stream_destroy": (C.c_int, [vp]),
        "chk_stream_add_tensor": (C.c_int, [vp, C.c_char_p, vp, u64, C.c_uint8]),
        "chk_stream_compress": (C.c_int, [vp]),
        "chk_stream_restore": (C.c_int, [vp, C.POINTER(vp)]),
        "chk_stream_part_count": (C.c_int, [vp, C.POINTER(u64)]),
        "chk_stream_part_info": (C.c_int, [vp, u64, C.POINTER(u64), C.POINTER(u64)]),
        "chk_stream_get_image": (C.c_int, [vp, u64, C.c_int, C.POINTER(vp), C.POINTER(u64)]),
        "chk_stream_get_summary": (C.c_int, [vp, C.POINTER(Summary)]),
        "chk_stream_save": (C.c_int, [vp, C.c_char_p]),
        "chk_stream_load": (C.c_int, [vp, C.c_char_p]),
        "chk_stream_get_timing": (C.c_int, [vp, C.c_char_p, C.POINTER(C.c_double)]),
        "chk_encode_tensor_static": (C.c_int, [vp, u64, C.c_uint8, u32p, u32p, vp, vp, C.POINTER(u64),
                                               C.POINTER(C.c_int), vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(rc):
    if rc != CHK_OK:
        raise CheckersError(rc, lib.chk_last_error().decode(errors="replace"))
