"""ctypes binding of libmk_b200.so (the C ABI declared in include/mk_cuda.h).

There is no CPU fallback: a missing library or a missing GPU raises.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "libmk_b200.so")

MK_OK = 0
MK_ERR_ARG, MK_ERR_CUDA, MK_ERR_OOM, MK_ERR_STATE, MK_ERR_TIMEOUT, MK_ERR_UNSUPPORTED = -1, -2, -3, -4, -5, -6
MK_ACT_Q8 = 0
MK_ACT_Q8X2 = 1
MK_ACT_FP4X6 = 2
MK_ACT_STRICT = 0x100
MK_SCALE_F32 = 0
MK_SCALE_F16 = 1
MK_MOE_SWIGLU_CLAMP = 0
MK_MOE_SITU = 1
MK_ROUTER_SIGMOID = 0
MK_ROUTER_SQRT_SOFTPLUS = 1
PROF_CATEGORIES = {"matvec_mxfp4": 0, "lm_head": 1, "router": 2, "experts": 3, "mla": 4, "other": 5}


class MkError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"libmk_b200 error {code}: {msg}")
        self.code = code


_lib = None

_vp = C.c_void_p
_i32 = C.c_int32
_i64 = C.c_int64

class KdaDesc(C.Structure):
    """mk_kda_desc"""
    _fields_ = [("heads", _i32), ("dim", _i32), ("kconv", _i32), ("gate_lb", C.c_float), ("rms_eps", C.c_float),
                ("q_conv", _vp), ("k_conv", _vp), ("v_conv", _vp), ("a_log", _vp), ("dt_bias", _vp), ("o_norm", _vp)]


class MoeDesc(C.Structure):
    """mk_moe_desc"""
    _fields_ = [("n_experts", _i32), ("top_k", _i32), ("d", _i32), ("inter", _i32),
                ("swiglu_limit", C.c_float), ("activation", _i32),
                ("gate_w", _vp), ("gate_b", _vp), ("experts", C.POINTER(_vp)), ("shared", _vp * 3),
                ("router", _i32), ("route_scale", C.c_float), ("latent", _i32), ("rms_eps", C.c_float),
                ("routed_down", _vp), ("routed_up", _vp), ("routed_norm", _vp), ("shared_f32", _vp * 3), ("act_mode", _i32)]


class MlaDesc(C.Structure):
    """mk_mla_desc"""
    _fields_ = [("layout", _i32), ("n_heads", _i32), ("nope", _i32), ("rope", _i32), ("vd", _i32),
                ("max_positions", _i32), ("n_seqs", _i32)]


class ModelConfig(C.Structure):
    """mk_model_config: the engine's Config (src/config.rs:8-43)."""
    _fields_ = ([(n, C.c_uint32) for n in ("n_layers", "d", "vocab", "n_experts", "top_k", "n_shared", "kda_heads", "kda_dim",
                                          "kda_conv", "kda_fa")] + [("gate_lb", C.c_float)] +
                [(n, C.c_uint32) for n in ("mla_heads", "mla_qa", "mla_kva", "mla_nope", "mla_rope", "mla_v", "routed_hidden",
                                          "moe_inter", "shared_inter", "dense_inter", "attn_res_block", "first_k_dense")] +
                [("rms_eps", C.c_float), ("eos_id", C.c_uint32), ("bos_id", C.c_uint32), ("has_layer_lists", C.c_uint32),
                 ("is_deepseek", C.c_uint32)])


class ModelOpts(C.Structure):
    """mk_model_opts"""
    _fields_ = [("max_positions", _i32), ("use_graph", _i32), ("strict", _i32), ("keep_layer_hidden", _i32), ("rank", _i32), ("world", _i32)]


_u32p = C.POINTER(C.c_uint32)
_u64p = C.POINTER(C.c_uint64)
_i32p = C.POINTER(_i32)

# name -> (restype, argtypes); every symbol include/mk_cuda.h declares
SIGNATURES = {
    "mk_init": (_i32, [_i32, C.POINTER(_vp)]),
    "mk_shutdown": (_i32, [_vp]),
    "mk_last_error": (C.c_char_p, []),
    "mk_set_stream": (_i32, [_vp, _vp]),
    "mk_sync": (_i32, [_vp]),
    "mk_memcpy_dev": (_i32, [_vp, _vp, _vp, C.c_uint64]),
    "mk_launch_count": (_i64, [_vp]),
    "mk_device_info": (_i32, [_vp, C.POINTER(_i32), C.POINTER(_i32), C.POINTER(_i32), C.POINTER(C.c_uint64)]),
    "mk_status_word": (_i32, [_vp, C.POINTER(_i32)]),
    "mk_set_option": (_i32, [_vp, C.c_char_p, _i64]),
    "mk_prof_enable": (_i32, [_vp, _i32]),
    "mk_prof_read": (_i32, [_vp, _i32, C.POINTER(_i64), C.POINTER(C.c_double)]),
    "mk_weight_mxfp4": (_i32, [_vp, _vp, _vp, _i64, _i64, _i32, C.POINTER(_vp)]),
    "mk_weight_q8_from_f32": (_i32, [_vp, _vp, _i64, _i64, _i32, _i32, C.POINTER(_vp)]),
    "mk_weight_q8": (_i32, [_vp, _vp, _vp, _i64, _i64, _i32, _i32, C.POINTER(_vp)]),
    "mk_weight_free": (_i32, [_vp, _vp]),
    "mk_weight_bytes": (_i64, [_vp]),
    "mk_weight_export": (_i32, [_vp, _vp, _vp, _vp]),
    "mk_dequant_mxfp4": (_i32, [_vp, _vp, _vp]),
    "mk_quantize_q8": (_i32, [_vp, _vp, _i64, _vp, _vp]),
    "mk_dequant_mxfp4_blob": (_i32, [_vp, _i32, _vp, _i64, _i64, _vp]),
    "mk_matvec_mxfp4": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32]),
    "mk_matvec_mxfp4_dev": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32]),
    "mk_gather_create": (_i32, [_vp, _i32, _i32, _i64, _i32, C.POINTER(_vp), _vp]),
    "mk_gather_connect": (_i32, [_vp, _vp, _vp]),
    "mk_gather_free": (_i32, [_vp, _vp]),
    "mk_matvec_q8_gather_dev": (_i32, [_vp, _vp, _vp, _vp, _i32, _i64, C.POINTER(_vp), _vp]),
    "mk_matvec_q8_gather_token_dev": (_i32, [_vp, _vp, _vp, _vp, _i32, _i64, C.POINTER(_vp), _vp]),
    "mk_dequant_fp8": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "mk_weight_vq1": (_i32, [_vp, _vp, _vp, _i64, _i64, _i32, C.POINTER(_vp)]),
    "mk_matvec_vq1": (_i32, [_vp, _vp, _vp, _vp, _i32]),
    "mk_matvec_vq1_dev": (_i32, [_vp, _vp, _vp, _vp, _i32]),
    "mk_weight_f32": (_i32, [_vp, _vp, _i64, _i64, _i32, C.POINTER(_vp)]),
    "mk_matvec_f32": (_i32, [_vp, _vp, _vp, _vp, _i32]),
    "mk_matvec_f32_dev": (_i32, [_vp, _vp, _vp, _vp, _i32]),
    "mk_rmsnorm_dev": (_i32, [_vp, _vp, _vp, _i32, _i32, C.c_float, _vp]),
    "mk_sigmoid_gate_dev": (_i32, [_vp, _vp, _vp, _i64]),
    "mk_kda_create": (_i32, [_vp, C.POINTER(KdaDesc), C.POINTER(_vp)]),
    "mk_kda_free": (None, [_vp, _vp]),
    "mk_kda_reset": (_i32, [_vp, _vp]),
    "mk_kda_step_dev": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mk_kda_steps_dev": (_i32, [_vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64]),
    "mk_kda_export": (_i32, [_vp, _vp, _vp, _vp]),
    "mk_kda_import": (_i32, [_vp, _vp, _vp, _vp]),
    "mk_attn_res_dev": (_i32, [_vp, _vp, _vp, _i64, _i32, _vp, _i32, C.c_float, _vp]),
    "mk_matvec_mxfp4_noalloc_dev": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32]),
    "mk_matvec_q8": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _vp]),
    "mk_matvec_q8_dev": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _vp]),
    "mk_moe_create": (_i32, [_vp, C.POINTER(MoeDesc), C.POINTER(_vp)]),
    "mk_moe_free": (_i32, [_vp, _vp]),
    "mk_moe_route": (_i32, [_vp, _vp, _vp, _i32, _vp, _vp, _vp]),
    "mk_moe_route_dev": (_i32, [_vp, _vp, _vp, _i32, _vp, _vp, _vp]),
    "mk_moe_forward": (_i32, [_vp, _vp, _vp, _i32, _vp, _vp, _vp]),
    "mk_moe_forward_dev": (_i32, [_vp, _vp, _vp, _i32, _vp, _vp, _vp]),
    "mk_moe_ep_create": (_i32, [_vp, _vp, _i32, _i32, _i32, C.POINTER(_vp), _vp]),
    "mk_moe_ep_connect": (_i32, [_vp, _vp, _vp]),
    "mk_moe_ep_free": (_i32, [_vp, _vp]),
    "mk_moe_forward_ep_dev": (_i32, [_vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp]),
    "mk_moe_experts_dev": (_i32, [_vp, _vp, _vp, _i32, _vp, _vp, _vp, _i32, _vp]),
    "mk_moe_combine_dev": (_i32, [_vp, _vp, _i32, _i32, _i32, _vp]),
    "mk_mla_create": (_i32, [_vp, C.POINTER(MlaDesc), C.POINTER(_vp)]),
    "mk_mla_free": (_i32, [_vp, _vp]),
    "mk_mla_reset": (_i32, [_vp, _vp, _i32]),
    "mk_mla_positions": (_i32, [_vp, _vp, _i32]),
    "mk_mla_append": (_i32, [_vp, _vp, _i32, _vp, _vp, _i32]),
    "mk_mla_append_dev": (_i32, [_vp, _vp, _i32, _vp, _vp, _i32]),
    "mk_mla_attend": (_i32, [_vp, _vp, _i32, _vp, _i32, C.c_float, _vp]),
    "mk_mla_attend_batch_dev": (_i32, [_vp, _vp, _vp, C.c_float, _vp]),
    "mk_mla_export": (_i32, [_vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp]),
    "mk_mla_export_f32": (_i32, [_vp, _vp, _i32, _vp, _vp]),
    "mk_mla_import_f32": (_i32, [_vp, _vp, _i32, _vp, _vp, _i32]),
    "mk_mla_decode_step_dev": (_i32, [_vp, _vp, _i32, _vp, _vp, _vp, C.c_float, _vp]),
    "mk_mla_prefill_dev": (_i32, [_vp, _vp, _i32, _vp, _vp, _vp, _i32, C.c_float, _vp]),
    "mk_model_config_default": (None, [C.POINTER(ModelConfig)]),
    "mk_bin_open": (_i32, [C.c_char_p, C.POINTER(_vp)]),
    "mk_bin_close": (_i32, [_vp]),
    "mk_bin_config": (_i32, [_vp, C.POINTER(ModelConfig)]),
    "mk_bin_count": (_i64, [_vp]),
    "mk_bin_find": (_i32, [_vp, C.c_char_p, _i32p, _i32p, _u32p, C.POINTER(_vp), _u64p]),
    "mk_bin_entry": (_i32, [_vp, _i64, C.POINTER(C.c_char_p), _i32p, _i32p, _u32p, C.POINTER(_vp), _u64p]),
    "mk_bin_writer_create": (_i32, [C.POINTER(ModelConfig), C.POINTER(_vp)]),
    "mk_bin_writer_add": (_i32, [_vp, C.c_char_p, _i32, _i32, _u32p]),
    "mk_bin_writer_begin": (_i32, [_vp, C.c_char_p]),
    "mk_bin_writer_put": (_i32, [_vp, C.c_char_p, _vp, C.c_uint64]),
    "mk_bin_writer_finish": (_i32, [_vp]),
    "mk_quantize_mxfp4_dev": (_i32, [_vp, _vp, _i64, _i64, _i32, _vp, _vp]),
    "mk_model_open": (_i32, [_vp, _vp, C.POINTER(ModelOpts), C.POINTER(_vp)]),
    "mk_model_free": (_i32, [_vp, _vp]),
    "mk_model_reset": (_i32, [_vp, _vp]),
    "mk_model_positions": (_i32, [_vp, _vp]),
    "mk_model_weight_bytes": (_i64, [_vp]),
    "mk_model_launches_per_token": (_i64, [_vp]),
    "mk_model_ep_handles": (_i32, [_vp, _vp, _vp]),
    "mk_model_ep_connect": (_i32, [_vp, _vp, _vp]),
    "mk_model_forward_dev": (_i32, [_vp, _vp, _vp, _vp, _vp]),
    "mk_model_forward": (_i32, [_vp, _vp, _i32, _vp, _vp]),
    "mk_model_prefill": (_i32, [_vp, _vp, _vp, _i32, _vp, _vp]),
    "mk_model_generate": (_i32, [_vp, _vp, _vp, _i32, _i32, _vp]),
    "mk_model_last_hidden": (_i32, [_vp, _vp, _vp]),
    "mk_model_layer_hidden": (_i32, [_vp, _vp, _vp]),
}


def load():
    """Loads the shared library (no GPU needed for this step)."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise ImportError(
                f"{SO_PATH} is missing: build it with `python -m microkimi_b200._build` "
                "(nvcc, sm_100a). There is no CPU fallback.")
        lib = C.CDLL(SO_PATH)
        for name, (res, args) in SIGNATURES.items():
            f = getattr(lib, name)
            f.restype = res
            f.argtypes = args
        _lib = lib
    return _lib


def check(rc):
    if rc != MK_OK:
        raise MkError(rc, load().mk_last_error().decode(errors="replace"))
