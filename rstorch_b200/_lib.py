"""ctypes binding of librstorch_b200.so (declarations in include/rstorch_b200.h).

The library is the only compute path: if it is missing, or a call fails, an
exception is raised.  Nothing here falls back to numpy or torch.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "librstorch_b200.so")
COMM_ID_BYTES = 128

STATUS_NAMES = {
    0: "RST_OK", 1: "RST_ERR_INVALID_ARG", 2: "RST_ERR_SHAPE", 3: "RST_ERR_FOREIGN_HANDLE",
    4: "RST_ERR_OOM", 5: "RST_ERR_CUDA", 6: "RST_ERR_NCCL", 7: "RST_ERR_DEVICE_TIMEOUT",
    8: "RST_ERR_NAN", 9: "RST_ERR_UNSUPPORTED", 10: "RST_ERR_STATE",
}
RST_OK, RST_ERR_INVALID_ARG, RST_ERR_SHAPE, RST_ERR_FOREIGN_HANDLE = 0, 1, 2, 3
RST_ERR_OOM, RST_ERR_CUDA, RST_ERR_NCCL, RST_ERR_DEVICE_TIMEOUT = 4, 5, 6, 7
RST_ERR_NAN, RST_ERR_UNSUPPORTED, RST_ERR_STATE = 8, 9, 10


class RstError(RuntimeError):
    """A C-ABI call returned a non-zero status (the reference panics in these cases)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status
        self.message = message


P = C.c_void_p
PP = C.POINTER(C.c_void_p)
I64 = C.c_int64
U64 = C.c_uint64
DBL = C.c_double
PD = C.POINTER(C.c_double)

# name -> (argtypes); every function returns int unless listed in _RESTYPES
_SIGNATURES = {
    "rst_version": [],
    "rst_status_string": [C.c_int],
    "rst_last_error": [P],
    "rst_ctx_create": [C.c_int, PP],
    "rst_ctx_destroy": [P],
    "rst_ctx_synchronize": [P],
    "rst_ctx_device": [P, C.POINTER(C.c_int)],
    "rst_ctx_stream": [P, PP],
    "rst_ctx_check_device": [P],
    "rst_selftest_wait_expiry": [P, I64],
    "rst_ctx_launch_count": [P, C.POINTER(U64)],
    "rst_ctx_memory_stats": [P, C.POINTER(U64)],
    "rst_ctx_set_memory_limit": [P, U64],
    "rst_ctx_empty_cache": [P],
    "rst_tensor_alloc": [P, I64, I64, PP],
    "rst_tensor_slice": [P, I64, I64, I64, PP],
    "rst_tensor_free": [P],
    "rst_tensor_shape": [P, C.POINTER(I64), C.POINTER(I64)],
    "rst_tensor_data": [P, PP],
    "rst_tensor_upload": [P, P],
    "rst_tensor_download": [P, P],
    "rst_tensor_copy": [P, P],
    "rst_tensor_fill": [P, DBL],
    "rst_tensor_checksum": [P, C.POINTER(U64)],
    "rst_linear_forward": [P, P, P, P, C.c_int, P],
    "rst_linear_backward": [P, P, P, P, P, P, P, P],
    "rst_linear_backward_chain": [P, C.c_int, P, P, P, P, P, P, P],
    "rst_linear_backward_t": [P, P, P, P, P, P, P, P, P, P],
    "rst_transpose": [P, P, P],
    "rst_bias_grad_noalloc": [P, I64, I64, P, P],
    "rst_relu_forward": [P, P, P],
    "rst_relu_backward": [P, P, P, P],
    "rst_softmax": [P, P, P],
    "rst_softmax_axis0": [P, P, P],
    "rst_softmax_backward": [P, P, P, P],
    "rst_xent_slots": [],
    "rst_xent_forward_backward": [P, P, P, P, C.c_int],
    "rst_xent_result": [P, C.c_int, PD, PD],
    "rst_accuracy": [P, P, P, PD],
    "rst_argmax": [P, P, C.POINTER(I64)],
    "rst_sgd_plan_create": [P, C.c_int, PP, PP, PP],
    "rst_sgd_plan_step": [P, DBL],
    "rst_sgd_plan_destroy": [P],
    "rst_sgd_step": [P, C.c_int, PP, PP, DBL],
    "rst_stager_create": [P, I64, I64, I64, C.c_int, PP],
    "rst_stager_destroy": [P],
    "rst_stager_host": [P, C.c_int, C.POINTER(PD), C.POINTER(PD)],
    "rst_stager_submit": [P, C.c_int],
    "rst_stager_acquire": [P, C.c_int, PP, PP],
    "rst_dataset_create_u8": [P, P, P, I64, I64, I64, PP],
    "rst_dataset_destroy": [P],
    "rst_dataset_len": [P, C.POINTER(I64)],
    "rst_dataset_gather": [P, C.POINTER(I64), I64, P, P],
    "rst_dataset_index_stage": [P, I64, C.POINTER(C.POINTER(I64))],
    "rst_dataset_gather_staged": [P, I64, P, P],
    "rst_dataset_shuffle": [P, U64],
    "rst_dataset_gather_epoch": [P, I64, I64, P, P],
    "rst_dataset_epoch_order": [P, C.POINTER(I64)],
    "rst_comm_get_id": [P],
    "rst_comm_create": [P, P, C.c_int, C.c_int, PP],
    "rst_comm_destroy": [P],
    "rst_allreduce_avg": [P, C.c_int, PP],
    "rst_comm_join": [P],
    "rst_comm_share_gradients": [P, C.c_int],
    "rst_graph_capture_begin": [P],
    "rst_graph_capture_end": [P, PP],
    "rst_graph_launch": [P],
    "rst_graph_destroy": [P],
    "rst_timer_create": [P, PP],
    "rst_timer_start": [P],
    "rst_timer_stop": [P],
    "rst_timer_elapsed_ms": [P, PD],
    "rst_timer_destroy": [P],
    "rst_synth_uniform": [U64, U64, U64, PD],
    "rst_synth_normal": [U64, U64, U64, DBL, DBL, PD],
    "rst_profile_begin": [P],
    "rst_profile_end": [P, C.c_char_p, C.c_size_t],
    "rst_probe_fp64_peak": [P, C.c_int, C.c_int, PD],
    "rst_probe_hbm_copy": [P, U64, C.c_int, PD],
    "rst_flush_l2": [P, U64],
}
_RESTYPES = {"rst_status_string": C.c_char_p, "rst_last_error": C.c_char_p}

_lib = None


def exported_symbols() -> list[str]:
    """Names every build of the library must export (one per declaration in the header)."""
    return sorted(_SIGNATURES)


def load() -> C.CDLL:
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m rstorch_b200.build` "
            "(there is no CPU or PyTorch fallback for the training step)")
    lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError = symbol missing = broken build
        fn.argtypes = argtypes
        fn.restype = _RESTYPES.get(name, C.c_int)
    _lib = lib
    return lib


def check(status: int, ctx_handle=None) -> None:
    if status != 0:
        msg = load().rst_last_error(ctx_handle)
        raise RstError(status, msg.decode("utf-8", "replace") if msg else "")
