"""ctypes binding of libllaisys.so: enums, handle types and the prototype of every exported symbol.

Mirrors the reference's binding package (python/llaisys/libllaisys/__init__.py:17-40 and its tensor.py,
ops.py, runtime.py, llaisys_types.py): the library sits next to this file and is loaded at import time, and
every prototype is declared immediately, so a missing symbol fails the import rather than a later call.
There is no pure-Python or CPU stand-in: without the compiled library the import raises.
"""
from __future__ import annotations

import ctypes
import sys
from ctypes import (CFUNCTYPE, POINTER, Structure, c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_size_t,
                    c_ssize_t, c_uint8, c_void_p)
from enum import IntEnum
from pathlib import Path


class DeviceType(IntEnum):
    CPU = 0
    NVIDIA = 1
    COUNT = 2


class DataType(IntEnum):
    INVALID = 0
    BYTE = 1
    BOOL = 2
    I8 = 3
    I16 = 4
    I32 = 5
    I64 = 6
    U8 = 7
    U16 = 8
    U32 = 9
    U64 = 10
    F8 = 11
    F16 = 12
    F32 = 13
    F64 = 14
    C16 = 15
    C32 = 16
    C64 = 17
    C128 = 18
    BF16 = 19


class MemcpyKind(IntEnum):
    H2H = 0
    H2D = 1
    D2H = 2
    D2D = 3


class Status(IntEnum):
    """Return codes of the paged-KV entry points (include/llaisys/paged_kv.h)."""
    OK = 0
    INVALID = 1
    NO_PAGES = 2
    NO_SEQ = 3
    DEVICE = 4
    UNSUPPORTED = 5
    KERNEL = 6


llaisysDeviceType_t = c_int
llaisysDataType_t = c_int
llaisysMemcpyKind_t = c_int
llaisysStream_t = c_void_p
llaisysTensor_t = c_void_p
llaisysPagedKV_t = c_void_p


class LlaisysRuntimeAPI(Structure):
    """The twelve function pointers of include/llaisys/runtime.h, in order."""
    _fields_ = [
        ("get_device_count", CFUNCTYPE(c_int)),
        ("set_device", CFUNCTYPE(None, c_int)),
        ("device_synchronize", CFUNCTYPE(None)),
        ("create_stream", CFUNCTYPE(llaisysStream_t)),
        ("destroy_stream", CFUNCTYPE(None, llaisysStream_t)),
        ("stream_synchronize", CFUNCTYPE(None, llaisysStream_t)),
        ("malloc_device", CFUNCTYPE(c_void_p, c_size_t)),
        ("free_device", CFUNCTYPE(None, c_void_p)),
        ("malloc_host", CFUNCTYPE(c_void_p, c_size_t)),
        ("free_host", CFUNCTYPE(None, c_void_p)),
        ("memcpy_sync", CFUNCTYPE(None, c_void_p, c_void_p, c_size_t, llaisysMemcpyKind_t)),
        ("memcpy_async", CFUNCTYPE(None, c_void_p, c_void_p, c_size_t, llaisysMemcpyKind_t, llaisysStream_t)),
    ]


_T = llaisysTensor_t
_KV = llaisysPagedKV_t
_I32P = POINTER(c_int32)

# name -> (restype, argtypes). Every symbol declared in include/llaisys/*.h appears here exactly once.


class LlaisysQwen2Meta(Structure):
    """struct LlaisysQwen2Meta (reference: include/llaisys/models/qwen2.h:7-13)."""
    _fields_ = [("dtype", llaisysDataType_t), ("nlayer", c_size_t), ("hs", c_size_t), ("nh", c_size_t),
                ("nkvh", c_size_t), ("dh", c_size_t), ("di", c_size_t), ("maxseq", c_size_t), ("voc", c_size_t),
                ("epsilon", c_float), ("theta", c_float), ("end_token", c_int64)]


class LlaisysQwen2Weights(Structure):
    """struct LlaisysQwen2Weights (reference: include/llaisys/models/qwen2.h:15-31)."""
    _fields_ = [("in_embed", llaisysTensor_t), ("out_embed", llaisysTensor_t), ("out_norm_w", llaisysTensor_t)] + [
        (name, POINTER(llaisysTensor_t)) for name in (
            "attn_norm_w", "attn_q_w", "attn_q_b", "attn_k_w", "attn_k_b", "attn_v_w", "attn_v_b", "attn_o_w",
            "mlp_norm_w", "mlp_gate_w", "mlp_up_w", "mlp_down_w")]


class LlaisysEngineEvent(Structure):
    """struct LlaisysEngineEvent (include/llaisys/serving.h)."""
    _fields_ = [("request", c_int64), ("token", c_int64), ("finished", c_int32), ("reserved", c_int32)]


_MODEL = c_void_p
ALL_REDUCE_FN = CFUNCTYPE(c_int, c_void_p, c_size_t, c_int, c_void_p)  # llaisysAllReduceFn

PROTOTYPES: dict[str, tuple] = {
    # runtime.h
    "llaisysGetRuntimeAPI": (POINTER(LlaisysRuntimeAPI), [llaisysDeviceType_t]),
    "llaisysSetContextRuntime": (None, [llaisysDeviceType_t, c_int]),
    "llaisysGetContextStream": (llaisysStream_t, []),
    # tensor.h
    "tensorCreate": (_T, [POINTER(c_size_t), c_size_t, llaisysDataType_t, llaisysDeviceType_t, c_int]),
    "tensorDestroy": (None, [_T]),
    "tensorGetData": (c_void_p, [_T]),
    "tensorGetNdim": (c_size_t, [_T]),
    "tensorGetShape": (None, [_T, POINTER(c_size_t)]),
    "tensorGetStrides": (None, [_T, POINTER(c_ssize_t)]),
    "tensorGetDataType": (llaisysDataType_t, [_T]),
    "tensorGetDeviceType": (llaisysDeviceType_t, [_T]),
    "tensorGetDeviceId": (c_int, [_T]),
    "tensorDebug": (None, [_T]),
    "tensorIsContiguous": (c_uint8, [_T]),
    "tensorLoad": (None, [_T, c_void_p]),
    "tensorView": (_T, [_T, POINTER(c_size_t), c_size_t]),
    "tensorPermute": (_T, [_T, POINTER(c_size_t)]),
    "tensorSlice": (_T, [_T, c_size_t, c_size_t, c_size_t]),
    # ops.h
    "llaisysAdd": (None, [_T, _T, _T]),
    "llaisysArgmax": (None, [_T, _T, _T]),
    "llaisysEmbedding": (None, [_T, _T, _T]),
    "llaisysLinear": (None, [_T, _T, _T, _T]),
    "llaisysLinearAccumulate": (None, [_T, _T, _T]),
    "llaisysRearrange": (None, [_T, _T]),
    "llaisysRmsNorm": (None, [_T, _T, _T, c_float]),
    "llaisysROPE": (None, [_T, _T, _T, c_float]),
    "llaisysSelfAttention": (None, [_T, _T, _T, _T, c_float]),
    "llaisysSwiGLU": (None, [_T, _T, _T]),
    # paged_kv.h
    "llaisysGetLastError": (c_char_p, []),
    "llaisysPagedKVCreate": (c_int, [POINTER(_KV), llaisysDeviceType_t, c_int, llaisysDataType_t, c_size_t, c_size_t,
                                     c_size_t, c_size_t, c_size_t, c_size_t, c_size_t]),
    "llaisysPagedKVDestroy": (c_int, [_KV]),
    "llaisysPagedKVSeqAdd": (c_int, [_KV, _I32P]),
    "llaisysPagedKVSeqReserve": (c_int, [_KV, c_int32, c_size_t]),
    "llaisysPagedKVSeqAssignPages": (c_int, [_KV, c_int32, _I32P, c_size_t]),
    "llaisysPagedKVSeqFree": (c_int, [_KV, c_int32]),
    "llaisysPagedKVNumFreePages": (c_size_t, [_KV]),
    "llaisysPagedKVNumSeqs": (c_size_t, [_KV]),
    "llaisysPagedKVSeqNumPages": (c_int64, [_KV, c_int32]),
    "llaisysPagedKVSeqPages": (c_int, [_KV, c_int32, _I32P, c_size_t]),
    "llaisysPagedKVPoolData": (c_void_p, [_KV, c_size_t]),
    "llaisysPagedKVLayerBytes": (c_size_t, [_KV]),
    "llaisysPagedKVBlockTableData": (c_void_p, [_KV]),
    "llaisysPagedKVFlush": (c_int, [_KV]),
    "llaisysPagedKVSetLaunchOverlap": (c_int, [_KV, c_int]),
    "llaisysPagedKVCheck": (c_int, [_KV]),
    "llaisysPagedKVAppend": (c_int, [_KV, c_size_t, c_void_p, c_void_p, _I32P, _I32P, c_size_t]),
    "llaisysPagedKVGather": (c_int, [_KV, c_size_t, c_int32, c_size_t, c_void_p, c_void_p]),
    "llaisysPagedAttentionDecode": (c_int, [_KV, c_size_t, c_void_p, c_void_p, _I32P, _I32P, c_size_t, c_size_t,
                                            c_float]),
    "llaisysPagedAttentionPrefill": (c_int, [_KV, c_size_t, c_void_p, c_void_p, _I32P, _I32P, _I32P, c_size_t,
                                             c_size_t, c_float]),
    "llaisysPagedAttentionDecodePartial": (c_int, [_KV, c_size_t, c_void_p, c_void_p, _I32P, _I32P, c_size_t,
                                                   c_size_t, c_float]),
    "llaisysLseMerge": (c_int, [llaisysDeviceType_t, c_int, c_void_p, llaisysDataType_t, c_void_p, c_size_t,
                                c_size_t, c_size_t]),
    "llaisysPagedKVAppendDev": (c_int, [_KV, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                        llaisysStream_t]),
    "llaisysPagedDecodeStepHost": (c_int, [_KV, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                           c_size_t, c_float]),
    "llaisysPagedKVSeqPublish": (c_int, [_KV, c_int32, POINTER(c_int64), c_size_t]),
    "llaisysPagedKVSeqMatchPrefix": (c_int, [_KV, c_int32, POINTER(c_int64), c_size_t, POINTER(c_size_t)]),
    "llaisysPagedKVSeqFork": (c_int, [_KV, c_int32, c_size_t, _I32P]),
    "llaisysPagedKVPageRefCount": (c_int, [_KV, c_int32]),
    "llaisysPagedKVNumCachedPages": (c_size_t, [_KV]),
    "llaisysPagedKVRopeAppendDev": (c_int, [_KV, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                            c_size_t, c_float, llaisysStream_t]),
    "llaisysPagedAttentionDecodeDev": (c_int, [_KV, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                               c_size_t, c_size_t, c_float, llaisysStream_t]),
    "llaisysPagedAttentionDecodePartialDev": (c_int, [_KV, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p,
                                                      c_size_t, c_size_t, c_size_t, c_float, llaisysStream_t]),
    "llaisysPagedAttentionPrefillDev": (c_int, [_KV, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                c_size_t, c_size_t, c_size_t, c_size_t, c_size_t, c_float,
                                                llaisysStream_t]),
    "llaisysPagedAttentionDecodeNoAlloc": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_size_t,
                                                   c_void_p, c_void_p, c_size_t, c_size_t, c_size_t, c_size_t,
                                                   llaisysDataType_t, c_float, c_void_p, llaisysStream_t]),
    "llaisysPeerExchangeCreate": (c_int, [POINTER(c_void_p), c_int, c_int, c_int, c_size_t]),
    "llaisysPeerExchangeDestroy": (None, [c_void_p]),
    "llaisysPeerExchangeHandle": (c_int, [c_void_p, c_void_p]),
    "llaisysPeerExchangeConnect": (c_int, [c_void_p, c_void_p]),
    "llaisysPagedAttentionDecodeSplitDev": (c_int, [_KV, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                                    c_size_t, c_size_t, c_float, c_void_p, llaisysStream_t]),
    "llaisysPeerExchangeStatus": (c_int, [c_void_p, llaisysStream_t]),
    "llaisysPeerExchangeSetWaitLimit": (c_int, [c_void_p, ctypes.c_uint32]),
    "llaisysPeerExchangeDisconnect": (c_int, [c_void_p]),
    "llaisysPagedDecodeStepDev": (c_int, [_KV, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_size_t, c_size_t, c_size_t, c_float, llaisysStream_t]),
    "llaisysPagedKVLastKernel": (c_int, [_KV]),
    "llaisysLastAttentionKernel": (c_int, []),
    "llaisysPagedAttentionDecodeNoAllocStatus": (c_int, [c_int, llaisysStream_t, _I32P]),
    "llaisysSetLinearPolicy": (c_int, [c_int]),
    # include/llaisys/models/qwen2.h
    "llaisysQwen2ModelCreate": (_MODEL, [POINTER(LlaisysQwen2Meta), llaisysDeviceType_t, POINTER(c_int), c_int]),
    "llaisysQwen2ModelDestroy": (None, [_MODEL]),
    "llaisysQwen2ModelWeights": (POINTER(LlaisysQwen2Weights), [_MODEL]),
    "llaisysQwen2ModelInfer": (c_int64, [_MODEL, POINTER(c_int64), c_size_t]),
    "llaisysQwen2ModelConfigureCache": (c_int, [_MODEL, c_size_t, c_size_t]),
    "llaisysQwen2ModelSeqAdd": (c_int, [_MODEL, _I32P]),
    "llaisysQwen2ModelSeqAddWithPrefix": (c_int, [_MODEL, POINTER(c_int64), c_size_t, _I32P, POINTER(c_size_t)]),
    "llaisysQwen2ModelSeqFree": (c_int, [_MODEL, c_int32]),
    "llaisysQwen2ModelReset": (c_int, [_MODEL]),
    "llaisysQwen2ModelStep": (c_int, [_MODEL, _I32P, _I32P, c_size_t, POINTER(c_int64), POINTER(c_int64)]),
    "llaisysQwen2ModelDecodeLoop": (c_int, [_MODEL, _I32P, c_size_t, POINTER(c_int64), c_size_t, POINTER(c_int64)]),
    "llaisysQwen2ModelLastLogits": (c_int, [_MODEL, POINTER(c_float), c_size_t]),
    "llaisysQwen2ModelLastLoopMs": (c_double, [_MODEL]),
    "llaisysQwen2ModelCreateTP": (_MODEL, [POINTER(LlaisysQwen2Meta), llaisysDeviceType_t, c_int, c_int, c_int]),
    "llaisysNcclUniqueId": (c_int, [c_void_p]),
    "llaisysQwen2ModelSetAllReduceNccl": (c_int, [_MODEL, c_void_p]),
    "llaisysQwen2ModelSetAllReduceCallback": (c_int, [_MODEL, ALL_REDUCE_FN, c_void_p]),
    # include/llaisys/serving.h
    "llaisysEngineCreate": (c_int, [POINTER(c_void_p), _MODEL, c_size_t, c_size_t, c_size_t]),
    "llaisysEngineDestroy": (None, [c_void_p]),
    "llaisysEngineSubmit": (c_int, [c_void_p, POINTER(c_int64), c_size_t, c_size_t, c_int64, POINTER(c_int64)]),
    "llaisysEngineStep": (c_int, [c_void_p, POINTER(LlaisysEngineEvent), c_size_t, POINTER(c_size_t)]),
    "llaisysEngineCancel": (c_int, [c_void_p, c_int64]),
    "llaisysEngineNumWaiting": (c_size_t, [c_void_p]),
    "llaisysEngineNumRunning": (c_size_t, [c_void_p]),
    "llaisysEngineCounter": (c_size_t, [c_void_p, c_int]),
}


def library_path() -> Path:
    if sys.platform.startswith("linux"):
        name = "libllaisys.so"
    elif sys.platform == "win32":
        name = "llaisys.dll"
    elif sys.platform == "darwin":
        name = "llaisys.dylib"
    else:
        raise RuntimeError("Unsupported platform")
    return Path(__file__).parent / name


def load_shared_library() -> ctypes.CDLL:
    path = library_path()
    if not path.is_file():
        raise FileNotFoundError(
            f"Shared library not found: {path}. Build it with `python llaisys_b200/build.py`; "
            "there is no Python fallback for the compiled kernels.")
    lib = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError here = the library is older than this binding
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


LIB_LLAISYS = load_shared_library()

__all__ = [
    "LIB_LLAISYS", "PROTOTYPES", "LlaisysRuntimeAPI", "llaisysStream_t", "llaisysTensor_t", "llaisysPagedKV_t",
    "llaisysDataType_t", "DataType", "llaisysDeviceType_t", "DeviceType", "llaisysMemcpyKind_t", "MemcpyKind",
    "Status", "library_path", "LlaisysQwen2Meta", "LlaisysQwen2Weights", "LlaisysEngineEvent", "ALL_REDUCE_FN",
]
