"""ctypes binding of ``lib/libnatsl_b200.so`` (the C ABI declared in ``include/natsl_b200.h``).

There is no fallback: if the library has not been built, importing the ops raises.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "libnatsl_b200.so")

DT_BF16, DT_F32, DT_F16, DT_I32 = 0, 1, 2, 3
RULE_GDN, RULE_MAMBA = 0, 1
FLAG_DECAY_SKIPPED, FLAG_ATTN_OWN_CHUNK, FLAG_NO_TRAILING_QUIRK, FLAG_ATTN_MMA_SYNC = 1, 2, 4, 8
FLAG_ATTN_PERSISTENT = 32
FLAG_BWD_REFERENCE_COMPAT = 16
ATTN_BT = 128

_p, _i, _f = C.c_void_p, C.c_int, C.c_float

# name -> argtypes; every function returns int except natsl_last_error
PROTOTYPES = {
    "natsl_abi_version": [],
    "natsl_device_status": [],
    "natsl_bounded_wait_selftest": [_i, _p],
    "natsl_build_tables": [_p, _i, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p],
    "natsl_attn_fwd": [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _p],
    "natsl_attn_fwd_ex": [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _p],
    "natsl_attn_fwd_split": [_p, _p, _p, _p, _i, _i, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i,
                             _i, _f, _i, _p],
    "natsl_pack_selected_pairs": [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _p],
    "natsl_sp_prefix_states": [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p],
    "natsl_sp_segment_decay": [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p],
    "natsl_sp_state_combine": [_p, _p, _p, _i, _i, _i, _i, _i, _i, _p],
    "natsl_pack_selected_blocks": [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _p],
    "natsl_attn_dense_mask": [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p],
    "natsl_chunk_local_cumsum": [_p, _p, _i, _i, _i, _p],
    "natsl_gdn_chunk_prep": [_p, _p, _p, _p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p],
    "natsl_linear_fwd_h": [_i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _p],
    "natsl_linear_fwd_o": [_i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _f, _i, _p],
    "natsl_gdn_chunk_prep_ex": [_p, _p, _p, _p, _p, _i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p],
    "natsl_gdn_chunk_prep_tc": [_p, _p, _p, _p, _p, _i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p],
    "natsl_gdn_walk_fused": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _f, _i, _p],
    "natsl_gdn_walk_fused_vsplit": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _f, _i, _p],
    "natsl_mamba_walk_fused": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _f, _i, _p],
    "natsl_linear_recurrent_fwd": [_i, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _p],
    "natsl_linear_recurrent_step": [_i, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _f,
                                    _i, _i, _p],
    "natsl_attn_fwd_fp32": [_i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _p],
    "natsl_norm_gate_mix": [_p, _p, _p, _p, _i, _p, _p, _i, _p, C.c_long, _i, _f, _i, _p],
    "natsl_attn_bwd": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _p],
    "natsl_linear_bwd_pre": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _f, _i, _p],
    "natsl_linear_bwd_dh": [_i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _f, _p],
    "natsl_linear_bwd_state": [_i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p,
                               _i, _i, _i, _i, _i, _i, _f, _i, _p],
    "natsl_linear_bwd_intra": [_i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _p, _p, _p, _p, _p, _p, _p, _p,
                               _p, _p, _i, _i, _i, _i, _i, _i, _f, _i, _p],
    "natsl_linear_bwd_dg": [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p],
    "natsl_norm_gate_mix_bwd": [_p, _p, _p, _p, _i, _p, _p, _i, _p, _p, _p, _p, _p, _p, _i, C.c_long, _i, _f, _i, _p],
    "natsl_short_conv_fwd": [_p, _p, _p, _p, _i, _i, _i, _i, _i, _p],
    "natsl_short_conv_bwd": [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p],
    "natsl_rmsnorm_fwd": [_p, _p, _p, _i, _p, _p, C.c_long, _i, _f, _p],
    "natsl_rmsnorm_bwd": [_p, _p, _i, _p, _p, _p, _p, _i, C.c_long, _i, _f, _p],
    "natsl_swiglu_fwd": [_p, _p, _p, C.c_long, _p],
    "natsl_swiglu_bwd": [_p, _p, _p, _p, _p, C.c_long, _p],
    "natsl_block_mean": [_p, _p, _i, _i, _i, _i, _p],
    "natsl_xent_rows": [_p, _p, _p, C.c_long, _i, C.c_long, _f, _p],
    "natsl_gdn_fwd_noalloc": [_p, _p, _p, _p, _p, _i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _p],
}
NOALLOC_SCRATCH_BYTES = 32 << 20

_lib = None


class NatslError(RuntimeError):
    pass


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise NatslError(
            f"{LIB_PATH} is missing: build it with `python -m neuralattentionsearchlinear_b200.build` "
            "(needs nvcc). There is no CPU or PyTorch fallback for these ops.")
    lib = C.CDLL(LIB_PATH)
    lib.natsl_last_error.restype = C.c_char_p
    lib.natsl_last_error.argtypes = []
    for name, args in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = C.c_int
        fn.argtypes = args
    _lib = lib
    return lib


# kernels one successful call of an entry point launches (for launch accounting; entry points not listed launch one)
KERNELS_PER_CALL = {"natsl_build_tables": 2, "natsl_attn_bwd": 2, "natsl_gdn_fwd_noalloc": 3, "natsl_abi_version": 0,
                    "natsl_device_status": 0}
_launches = 0


def kernel_launches() -> int:
    """Number of kernels this process has launched through ``call`` so far."""
    return _launches


# NATSL_CHECK_STATUS=1: after every entry point, wait for the device and read the status word the kernels' bounded waits
# and capacity checks write (natsl_device_status); a non-zero word raises.  A debugging aid: it serialises host and device.
CHECK_STATUS = os.environ.get("NATSL_CHECK_STATUS", "0") == "1"
_DEVICE_STATUS_TEXT = {1: "a bounded wait inside a kernel ran out", 2: "a tensor-core kernel found its shared memory misaligned",
                       3: "a caller-given capacity was too small"}


def call(name: str, *args) -> None:
    global _launches
    lib = load()
    status = getattr(lib, name)(*args)
    _launches += KERNELS_PER_CALL.get(name, 1)
    if status != 0:
        raise NatslError(f"{name} failed with status {status}: {lib.natsl_last_error().decode()}")
    if CHECK_STATUS and name not in ("natsl_device_status", "natsl_abi_version", "natsl_bounded_wait_selftest"):
        import torch
        torch.cuda.synchronize()
        word = lib.natsl_device_status()
        if word != 0:
            raise NatslError(f"{name}: device status {word} ({_DEVICE_STATUS_TEXT.get(word, 'unknown')})")


def ptr(t) -> int | None:
    """Device pointer of a torch tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()
