"""ctypes binding of libsaf_b200.so (declared in include/saf_b200.h).

The library is the only compute path: if it is missing, importing this module
raises with the build command.  There is no Triton, no torch and no CPU fallback.
"""
import ctypes as C
import os

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.environ.get("SAF_B200_LIB") or os.path.join(_ROOT, "lib", "libsaf_b200.so")

SAF_OK, SAF_ERR_INVALID, SAF_ERR_UNSUPPORTED, SAF_ERR_CUDA, SAF_ERR_LIMIT = 0, -1, -2, -3, -4
SAF_F32, SAF_BF16, SAF_F16 = 0, 1, 2
LIVE, DENSE, DECOMP, SINK_DECAY = 0, 1, 2, 3
MAX_WEIGHTS = 4
STATIC_DELTA_FLOATS = 1 << 20


class SafTensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride", C.c_int64 * 4)]


class SafMixedAttnArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_int32), ("dtype", C.c_int32),
        ("B", C.c_int32), ("H", C.c_int32), ("U", C.c_int32), ("T", C.c_int32), ("HD", C.c_int32),
        ("HKV", C.c_int32), ("S", C.c_int32), ("SD", C.c_int32),
        ("patt_dtype", C.c_int32), ("dec_dtype", C.c_int32), ("rope", C.c_int32), ("force_state", C.c_int32),
        ("sm_scale", C.c_float),
        ("q", SafTensor), ("k", SafTensor), ("v", SafTensor), ("out", SafTensor), ("lse", SafTensor),
        ("patt", SafTensor), ("alpha", SafTensor), ("rho", SafTensor), ("z", SafTensor),
        ("frozen", C.c_void_p), ("hidx", C.c_void_p), ("pidx", C.c_void_p), ("kvidx", C.c_void_p),
        ("frozen_host", C.POINTER(C.c_int32)),
        ("sd_alpha", C.c_void_p), ("sd_rho", C.c_void_p), ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p),
        ("status", C.c_void_p), ("sched", C.c_void_p),
    ]


class SafMixedAttnBwdArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_int32), ("fwd", SafMixedAttnArgs),
        ("dout", SafTensor), ("dq", SafTensor), ("dk", SafTensor), ("dv", SafTensor), ("delta", SafTensor),
    ]


class SafFrozenPvArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_int32), ("dtype", C.c_int32), ("patt_dtype", C.c_int32),
        ("B", C.c_int32), ("NF", C.c_int32), ("T", C.c_int32), ("HD", C.c_int32), ("S", C.c_int32),
        ("patt", SafTensor), ("v", SafTensor), ("y", SafTensor),
        ("fz_idx", C.c_void_p), ("sd_alpha", C.c_void_p), ("sd_rho", C.c_void_p), ("status", C.c_void_p),
    ]


class SafIndexedLinearArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_int32), ("dtype", C.c_int32), ("M", C.c_int32), ("C", C.c_int32),
        ("n_weights", C.c_int32), ("n_slabs", C.c_int32), ("slab", C.c_int32), ("T", C.c_int32),
        ("x", C.c_void_p), ("ldx", C.c_int64),
        ("weights", C.c_void_p * MAX_WEIGHTS), ("biases", C.c_void_p * MAX_WEIGHTS),
        ("ldw", C.c_int64 * MAX_WEIGHTS), ("cdw", C.c_int64 * MAX_WEIGHTS), ("rows_w", C.c_int32 * MAX_WEIGHTS),
        ("slab_weight", C.POINTER(C.c_int32)), ("slab_row0", C.POINTER(C.c_int32)),
        ("slab_rope", C.POINTER(C.c_int32)),
        ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p),
        ("out", C.c_void_p), ("ldo", C.c_int64), ("status", C.c_void_p),
        ("act", C.c_int32), ("residual", C.c_void_p), ("ldr", C.c_int64),
    ]


class SafPatternGradArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_int32), ("dtype", C.c_int32),
        ("B", C.c_int32), ("H", C.c_int32), ("T", C.c_int32), ("HD", C.c_int32), ("SD", C.c_int32),
        ("force_state", C.c_int32),
        ("v", SafTensor), ("out", SafTensor), ("dout", SafTensor),
        ("alpha", C.c_void_p), ("rho", C.c_void_p), ("z", C.c_void_p),
        ("frozen", C.c_void_p), ("frozen_host", C.POINTER(C.c_int32)),
        ("dalpha", C.c_void_p), ("drho", C.c_void_p), ("delta", C.c_void_p), ("status", C.c_void_p),
    ]


class SafAttnStatsArgs(C.Structure):
    _fields_ = [
        ("struct_size", C.c_int32), ("dtype", C.c_int32),
        ("B", C.c_int32), ("U", C.c_int32), ("T", C.c_int32), ("HD", C.c_int32), ("sm_scale", C.c_float),
        ("q", SafTensor), ("k", SafTensor), ("lse", SafTensor),
        ("mean", C.c_void_p), ("count_prev", C.c_int64), ("head_m2", C.c_void_p), ("neg_entropy", C.c_void_p),
        ("status", C.c_void_p),
        ("quantity", C.c_int32), ("cell_m2", C.c_void_p),
    ]


STATS_PROBS, STATS_LOGITS = 0, 1
ACT_NONE, ACT_GELU, ACT_SWIGLU = 0, 1, 2

EXPORTS = (
    "saf_abi_version", "saf_last_error", "saf_launch_count", "saf_device_supported",
    "saf_mixed_attn_fwd", "saf_mixed_attn_bwd", "saf_mixed_attn_bwd_static", "saf_frozen_pv_fwd", "saf_frozen_pv_bwd",
    "saf_indexed_linear_fwd", "saf_indexed_linear_bwd_dx", "saf_indexed_linear_bwd_dw",
    "saf_decomposed_logz", "saf_rope_slabs", "saf_layernorm_fwd", "saf_rmsnorm_fwd",
    "saf_pattern_normalisers", "saf_pattern_param_grad", "saf_attention_moments",
    "saf_selftest_wait_timeout", "saf_selftest_per_device_once", "saf_selftest_mma_rate",
)


class SafError(RuntimeError):
    def __init__(self, code, text):
        super().__init__("libsaf_b200 error %d: %s" % (code, text))
        self.code = code


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "libsaf_b200.so is not built (%s). Build it with `python -m saf_b200.build` "
            "(needs nvcc); this package has no fallback path." % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    lib.saf_abi_version.restype = C.c_int
    lib.saf_last_error.argtypes = [C.c_char_p, C.c_size_t]
    lib.saf_last_error.restype = C.c_int
    lib.saf_launch_count.restype = C.c_int64
    lib.saf_device_supported.restype = C.c_int
    for name, at in (("saf_mixed_attn_fwd", SafMixedAttnArgs), ("saf_mixed_attn_bwd", SafMixedAttnBwdArgs),
                     ("saf_mixed_attn_bwd_static", SafMixedAttnBwdArgs),
                     ("saf_frozen_pv_fwd", SafFrozenPvArgs), ("saf_frozen_pv_bwd", SafFrozenPvArgs),
                     ("saf_indexed_linear_fwd", SafIndexedLinearArgs),
                     ("saf_pattern_param_grad", SafPatternGradArgs),
                     ("saf_attention_moments", SafAttnStatsArgs)):
        f = getattr(lib, name)
        f.argtypes = [C.POINTER(at), C.c_void_p]
        f.restype = C.c_int
    lib.saf_indexed_linear_bwd_dx.argtypes = [C.POINTER(SafIndexedLinearArgs), C.c_void_p, C.c_int64, C.c_void_p,
                                              C.c_int64, C.c_void_p, C.c_void_p]
    lib.saf_indexed_linear_bwd_dx.restype = C.c_int
    lib.saf_indexed_linear_bwd_dw.argtypes = [C.POINTER(SafIndexedLinearArgs), C.c_void_p, C.c_int64, C.c_void_p]
    lib.saf_indexed_linear_bwd_dw.restype = C.c_int
    lib.saf_decomposed_logz.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]
    lib.saf_decomposed_logz.restype = C.c_int
    lib.saf_pattern_normalisers.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                            C.c_void_p]
    lib.saf_pattern_normalisers.restype = C.c_int
    lib.saf_rope_slabs.argtypes = [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                   C.POINTER(C.c_int32), C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]
    lib.saf_rope_slabs.restype = C.c_int
    lib.saf_layernorm_fwd.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                      C.c_int32, C.c_int32, C.c_float, C.c_int32, C.c_void_p]
    lib.saf_layernorm_fwd.restype = C.c_int
    lib.saf_rmsnorm_fwd.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32,
                                    C.c_float, C.c_int32, C.c_void_p]
    lib.saf_rmsnorm_fwd.restype = C.c_int
    lib.saf_selftest_wait_timeout.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
    lib.saf_selftest_wait_timeout.restype = C.c_int
    lib.saf_selftest_mma_rate.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.saf_selftest_mma_rate.restype = C.c_int
    lib.saf_selftest_per_device_once.restype = C.c_int
    if lib.saf_abi_version() != 2:
        raise ImportError("libsaf_b200.so ABI version %d, expected 2: rebuild" % lib.saf_abi_version())
    return lib


lib = _load()


def last_error():
    buf = C.create_string_buffer(512)
    lib.saf_last_error(buf, 512)
    return buf.value.decode("utf-8", "replace")


def check(rc):
    if rc != SAF_OK:
        raise SafError(rc, last_error())
