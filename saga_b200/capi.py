"""ctypes binding of the b200opt C ABI (include/b200opt.h).

Loading fails loudly when libb200opt.so has not been built: there is no
fallback path of any kind.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200opt.so")

OK, EINVAL, ECUDA, ENOMEM, ETIMEOUT, ESTATE, EUNSUPPORTED, ETOOBIG = 0, -1, -2, -3, -4, -5, -6, -7
STATIC_MAX_ELEMS = 1 << 30
HALF, FLOAT = 0, 1
POLICY_REFERENCE, POLICY_INTERVAL = 0, 1
PATH_AUTO, PATH_PEER, PATH_NCCL, PATH_NVLS = 0, 1, 2, 3
OPT_TIMEOUT_MS, OPT_PATH, OPT_CTAS_PER_SM, OPT_KERNEL_VARIANT, OPT_NCCL_CROSSOVER = 1, 2, 3, 4, 5
OPT_STAGES, OPT_GRID, OPT_PHASE_TIMERS, OPT_ASSUME_NO_PEER_ACCESS, OPT_KEEP_REDUCED = 6, 7, 8, 9, 10
KERNEL_DIRECT, KERNEL_STAGED = 1, 2
CREATE_FABRIC, CREATE_MULTICAST = 1, 2
MAX_RANKS = 8
IPC_HANDLE_BYTES = 64
NCCL_ID_BYTES = 128

_vp, _sz, _i, _f = C.c_void_p, C.c_size_t, C.c_int, C.c_float
_u32p = C.POINTER(C.c_uint32)
_fp = C.POINTER(C.c_float)

# name -> (restype, argtypes); every function include/b200opt.h declares
SIGNATURES = {
    "b200opt_version": (C.c_char_p, []),
    "b200opt_strerror": (C.c_char_p, [_i]),
    "b200opt_last_error": (C.c_char_p, [_vp]),
    "b200opt_create": (_i, [C.POINTER(_vp), _i, _i, _i, _sz, _sz]),
    "b200opt_create_ex": (_i, [C.POINTER(_vp), _i, _i, _i, _sz, _sz, C.c_uint]),
    "b200opt_create_group": (_i, [C.POINTER(_vp), _i, C.POINTER(_i), _sz, _sz]),
    "b200opt_create_group_ex": (_i, [C.POINTER(_vp), _i, C.POINTER(_i), _sz, _sz, C.c_uint]),
    "b200opt_destroy": (_i, [_vp]),
    "b200opt_ipc_export": (_i, [_vp, _vp]),
    "b200opt_ipc_attach": (_i, [_vp, _i, _vp]),
    "b200opt_attach_local": (_i, [_vp, _i, _vp]),
    "b200opt_fd_export": (_i, [_vp, C.POINTER(_i)]),
    "b200opt_fd_attach": (_i, [_vp, _i, _i]),
    "b200opt_multicast_supported": (_i, [_i, C.POINTER(_i)]),
    "b200opt_mc_create": (_i, [_vp, C.POINTER(_i)]),
    "b200opt_mc_join": (_i, [_vp, _i]),
    "b200opt_mc_bind": (_i, [_vp]),
    "b200opt_nccl_unique_id": (_i, [_vp]),
    "b200opt_nccl_init": (_i, [_vp, _vp]),
    "b200opt_buffers": (_i, [_vp, _i, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_sz)]),
    "b200opt_layout": (_i, [C.POINTER(_sz), _sz, C.POINTER(_sz), C.POINTER(_sz)]),
    "b200opt_init_master": (_i, [_vp, _vp]),
    "b200opt_step": (_i, [_vp, _f, _f, _f, _vp]),
    "b200opt_step_begin": (_i, [_vp]),
    "b200opt_step_bucket": (_i, [_vp, _sz, _sz, _sz, _sz, _f, _f, _f, _vp, _i]),
    "b200opt_step_host": (_i, [_vp, _vp, _vp, _f, _f, _f, _vp, _u32p]),
    "b200opt_flags": (_i, [_vp, _vp, _u32p]),
    "b200opt_device_scale_enable": (_i, [_vp, _f, _i, _i, _sz]),
    "b200opt_device_scale_ptr": (_i, [_vp, C.POINTER(_vp)]),
    "b200opt_step_device_scale": (_i, [_vp, _f, _f, _vp]),
    "b200opt_device_scale_read": (_i, [_vp, _vp, _fp, _vp, _sz, C.POINTER(_sz)]),
    "b200opt_device_scale_peek": (_i, [_vp, _fp, _u32p]),
    "b200opt_policy_update": (_i, [_fp, _u32p, _i, C.POINTER(_i), _i]),
    "b200opt_bias_corrections": (_i, [_i, _fp, _fp]),
    "b200opt_choose_path": (_i, [_i, _i, _i, _i, _i, _i, _sz, _sz, C.POINTER(_i)]),
    "b200opt_adam_mixed": (_i, [_sz, _f, _vp, _vp, _vp, _vp, _vp, _f, _f, _f, _f, _vp, _vp]),
    "b200opt_adam_float": (_i, [_sz, _vp, _vp, _vp, _vp, _f, _f, _f, _f, _vp, _vp]),
    "b200opt_adam_mixed_static": (_i, [_sz, _f, _vp, _vp, _vp, _vp, _vp, _f, _f, _f, _f, _vp, _vp]),
    "b200opt_get_iter": (_i, [_vp, C.POINTER(_i)]),
    "b200opt_set_iter": (_i, [_vp, _i]),
    "b200opt_export_state": (_i, [_vp, _i, _i, _vp, _sz, C.POINTER(_sz)]),
    "b200opt_import_state": (_i, [_vp, _i, _i, _vp, _sz]),
    "b200opt_rank_info": (_i, [_vp, C.POINTER(_i), C.POINTER(_i)]),
    "b200opt_tensor_save": (_i, [C.c_char_p, _i, C.c_uint, _u32p, _vp]),
    "b200opt_tensor_load": (_i, [C.c_char_p, C.POINTER(_i), C.POINTER(C.c_uint), _u32p, _vp, _sz,
                                C.POINTER(_sz)]),
    "b200opt_checkpoint_save": (_i, [_vp, C.c_char_p, _f, _i]),
    "b200opt_checkpoint_load": (_i, [_vp, C.c_char_p, _fp, C.POINTER(_i)]),
    "b200opt_set_option": (_i, [_vp, _i, C.c_long]),
    "b200opt_get_option": (_i, [_vp, _i, C.POINTER(C.c_long)]),
    "b200opt_peer_copy": (_i, [_vp, _i, _sz, _vp]),
    "b200opt_phase_times": (_i, [_vp, C.POINTER(C.c_uint64)]),
    "b200opt_launch_count": (_i, [_vp, C.POINTER(C.c_uint64)]),
}

_lib = None


class B200OptError(RuntimeError):
    def __init__(self, status, detail=""):
        self.status = status
        name = lib().b200opt_strerror(status).decode()
        super().__init__(f"b200opt status {status} ({name})" + (f": {detail}" if detail else ""))


def lib():
    """Returns the loaded library; raises if it is missing (no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m saga_b200.build` "
                "(nvcc, sm_100a). saga_b200 has no CPU or PyTorch fallback.")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if a symbol is missing
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status, handle=None):
    if status != OK:
        detail = ""
        if handle:
            detail = lib().b200opt_last_error(handle).decode()
        raise B200OptError(status, detail)
