"""ctypes binding of libtlnn.so, the sm_100a engine.

There is no CPU path: if the shared library is missing or cannot be loaded, importing this module raises.  The
prototypes below are the declarations of ``include/tlnn.h``.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# TLNN_DEBUG=1 selects the debug build (device-side bounds checks compiled in): `python -m torchless_nn_b200.build --debug`
LIB_PATH = os.path.join(HERE, "libtlnn_debug.so" if os.environ.get("TLNN_DEBUG") == "1" else "libtlnn.so")

OK, ERR_VALUE, ERR_INDEX, ERR_CUDA, ERR_NOMEM, ERR_TIMEOUT, ERR_NULL = 0, -1, -2, -3, -4, -5, -6
F32, BF16, I32, I64, U8 = 0, 1, 2, 3, 4
PREC_TF32, PREC_BF16 = 0, 1
ACT_NONE, ACT_GELU, ACT_SILU, ACT_RELU = 0, 1, 2, 3

c_void_pp = C.POINTER(C.c_void_p)
ll = C.c_longlong
vp = C.c_void_p


class BlockParams(C.Structure):
    """tlnn_block_params: the twelve tensors of one TransformerBlock in registration order."""
    _fields_ = [(n, vp) for n in ("ln1_gamma", "ln1_beta", "wqkv_t", "bqkv", "wo_t", "bo",
                                  "ln2_gamma", "ln2_beta", "w1_t", "b1", "w2_t", "b2")]


class GPTModel(C.Structure):
    """tlnn_gpt_model."""
    _fields_ = [("vocab", C.c_int), ("context", C.c_int), ("d", C.c_int), ("heads", C.c_int), ("layers", C.c_int),
                ("act", C.c_int), ("prec", C.c_int),
                ("tok_table", vp), ("pos_table", vp), ("blocks", C.POINTER(BlockParams)),
                ("lnf_gamma", vp), ("lnf_beta", vp), ("head_t", vp), ("head_bias", vp)]


class ViTModel(C.Structure):
    """tlnn_vit_model."""
    _fields_ = [(n, C.c_int) for n in ("channels", "height", "width", "patch_h", "patch_w", "d", "heads", "layers", "act",
                                       "prec", "registers", "n_out")] + \
               [("proj_t", vp), ("cls_reg", vp), ("pos", vp), ("blocks", C.POINTER(BlockParams)),
                ("lnf_gamma", vp), ("lnf_beta", vp), ("head_t", vp), ("head_bias", vp)]


class ProfRow(C.Structure):
    _fields_ = [("name", C.c_char * 48), ("launches", ll), ("ms", C.c_double)]


# name -> (restype, argtypes); every symbol declared in include/tlnn.h
PROTOTYPES = {
    "tlnn_version": (C.c_int, []),
    "tlnn_init": (C.c_int, [C.c_int, c_void_pp]),
    "tlnn_shutdown": (C.c_int, [vp]),
    "tlnn_last_error": (C.c_char_p, []),
    "tlnn_sync": (C.c_int, [vp]),
    "tlnn_check": (C.c_int, [vp]),
    "tlnn_stream": (vp, [vp]),
    "tlnn_device_info": (C.c_int, [vp, C.POINTER(C.c_int), C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "tlnn_launch_count": (ll, [vp, C.c_int]),
    "tlnn_alloc": (C.c_int, [vp, C.c_size_t, c_void_pp]),
    "tlnn_free": (C.c_int, [vp, vp]),
    "tlnn_host_alloc": (C.c_int, [C.c_size_t, c_void_pp]),
    "tlnn_host_free": (C.c_int, [vp]),
    "tlnn_h2d": (C.c_int, [vp, vp, vp, C.c_size_t]),
    "tlnn_d2h": (C.c_int, [vp, vp, vp, C.c_size_t]),
    "tlnn_d2h_async": (C.c_int, [vp, vp, vp, C.c_size_t]),
    "tlnn_d2d": (C.c_int, [vp, vp, vp, C.c_size_t]),
    "tlnn_memset": (C.c_int, [vp, vp, C.c_int, C.c_size_t]),
    "tlnn_axpby_f32": (C.c_int, [vp, vp, C.c_float, vp, C.c_float, C.c_size_t]),
    "tlnn_add_f32": (C.c_int, [vp, vp, vp, vp, C.c_size_t]),
    "tlnn_gather_f32": (C.c_int, [vp, vp, vp, vp, C.c_size_t]),
    "tlnn_weight_prepare": (C.c_int, [vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, vp]),
    "tlnn_linear_fwd": (C.c_int, [vp, C.c_int, vp, ll, vp, vp, C.c_int, vp, ll, vp, ll, C.c_int, C.c_int, C.c_int]),
    "tlnn_embed_fwd": (C.c_int, [vp, vp, C.c_int, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int]),
    "tlnn_layernorm_fwd": (C.c_int, [vp, vp, vp, vp, C.c_float, vp, ll, C.c_int]),
    "tlnn_activation_fwd": (C.c_int, [vp, C.c_int, vp, vp, C.c_size_t]),
    "tlnn_softmax_fwd": (C.c_int, [vp, vp, vp, ll, C.c_int, C.c_float]),
    "tlnn_argmax_fwd": (C.c_int, [vp, vp, ll, vp, ll, C.c_int]),
    "tlnn_sample_fwd": (C.c_int, [vp, vp, ll, vp, vp, ll, C.c_int]),
    "tlnn_feed_create": (C.c_int, [vp, C.c_size_t, C.POINTER(vp)]),
    "tlnn_feed_host": (C.c_int, [vp, C.c_int, C.POINTER(vp)]),
    "tlnn_feed_host_wait": (C.c_int, [vp, C.c_int]),
    "tlnn_feed_submit": (C.c_int, [vp, C.c_int, C.c_size_t]),
    "tlnn_feed_acquire": (C.c_int, [vp, C.c_int, C.POINTER(vp)]),
    "tlnn_feed_release": (C.c_int, [vp, C.c_int]),
    "tlnn_feed_destroy": (C.c_int, [vp]),
    "tlnn_selftest_wait": (C.c_int, [vp, C.c_int]),
    "tlnn_eval_batch_fwd": (C.c_int, [vp, vp, ll, vp, C.c_int, ll, C.c_int, vp, vp]),
    "tlnn_attention_fwd": (C.c_int, [vp, C.c_int, vp, vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "tlnn_ffn_fwd": (C.c_int, [vp, C.c_int, vp, vp, vp, vp, vp, C.c_int, vp, ll, C.c_int]),
    "tlnn_block_fwd": (C.c_int, [vp, C.c_int, vp, C.POINTER(BlockParams), C.c_int, vp, C.c_int, C.c_int, C.c_int,
                                 C.c_int, C.c_int]),
    "tlnn_logits_fwd": (C.c_int, [vp, C.c_int, vp, vp, vp, vp, vp, ll, C.c_int, C.c_int]),
    "tlnn_norm_logits_fwd": (C.c_int, [vp, C.c_int, vp, vp, vp, vp, vp, vp, vp, ll, C.c_int, C.c_int]),
    "tlnn_logits_tokens_noalloc": (C.c_int, [vp, C.c_int, vp, vp, vp, vp, ll, C.c_int, C.c_int]),
    "tlnn_vit_project_fwd": (C.c_int, [vp, C.c_int, vp, vp, vp, vp, vp] + [C.c_int] * 8),
    "tlnn_vit_head_fwd": (C.c_int, [vp, C.c_int, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int]),
    "tlnn_vit_forward": (C.c_int, [vp, C.POINTER(ViTModel), vp, C.c_int, vp]),
    "tlnn_gpt_prefill": (C.c_int, [vp, C.POINTER(GPTModel), vp, C.c_int, C.c_int, C.c_int, vp, vp]),
    "tlnn_decode_begin": (C.c_int, [vp, C.POINTER(GPTModel), vp, C.c_int, C.c_int, C.c_int, C.c_int, vp, c_void_pp]),
    "tlnn_decode_step": (C.c_int, [vp, vp, vp]),
    "tlnn_decode_run": (C.c_int, [vp, vp, C.c_int, vp]),
    "tlnn_decode_first_sampled": (C.c_int, [vp, C.c_float, vp, vp]),
    "tlnn_decode_run_sampled": (C.c_int, [vp, vp, C.c_int, C.c_float, vp, vp]),
    "tlnn_decode_end": (C.c_int, [vp]),
    "tlnn_comm_nccl_version": (C.c_int, [C.POINTER(C.c_int)]),
    "tlnn_comm_unique_id": (C.c_int, [vp]),
    "tlnn_comm_init": (C.c_int, [vp, vp, C.c_int, C.c_int, c_void_pp]),
    "tlnn_comm_rank": (C.c_int, [vp, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "tlnn_allgather_tokens": (C.c_int, [vp, vp, vp, ll, C.POINTER(ll)]),
    "tlnn_allgather_logits": (C.c_int, [vp, vp, vp, ll, C.POINTER(ll)]),
    "tlnn_comm_barrier": (C.c_int, [vp]),
    "tlnn_comm_destroy": (C.c_int, [vp]),
    "tlnn_debug_canaries": (C.c_int, [vp, C.c_int]),
    "tlnn_debug_check": (C.c_int, [vp, C.POINTER(ll), C.POINTER(ll)]),
    "tlnn_prof_begin": (C.c_int, [vp]),
    "tlnn_prof_end": (C.c_int, [vp, C.POINTER(C.c_float)]),
    "tlnn_prof_classes": (C.c_int, [vp, C.c_int]),
    "tlnn_prof_table": (C.c_int, [vp, C.POINTER(ProfRow), C.c_int]),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m torchless_nn_b200.build` (needs nvcc). "
            "torchless_nn_b200 has no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)      # AttributeError here means the library and the header disagree
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def last_error() -> str:
    return lib.tlnn_last_error().decode("utf-8", "replace")


_EXC = {ERR_VALUE: ValueError, ERR_NULL: ValueError, ERR_INDEX: IndexError, ERR_CUDA: RuntimeError,
        ERR_NOMEM: MemoryError, ERR_TIMEOUT: RuntimeError}


def check(status: int):
    """Raise the Python exception class the reference would raise for the same misuse."""
    if status != OK:
        raise _EXC.get(status, RuntimeError)(f"libtlnn: {last_error()} (status {status})")
