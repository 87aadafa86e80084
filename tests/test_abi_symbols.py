"""The shared library loads without a GPU and exports every symbol the public headers declare."""
import ctypes
import re
from pathlib import Path

import llaisys_b200 as llaisys
from llaisys_b200 import libllaisys

INCLUDE = Path(__file__).resolve().parents[1] / "include"

# the 26 symbols of the reference ABI (reference: include/llaisys/{runtime,tensor,ops}.h)
REFERENCE_SYMBOLS = {
    "llaisysGetRuntimeAPI", "llaisysSetContextRuntime",
    "tensorCreate", "tensorDestroy", "tensorGetData", "tensorGetNdim", "tensorGetShape", "tensorGetStrides",
    "tensorGetDataType", "tensorGetDeviceType", "tensorGetDeviceId", "tensorDebug", "tensorIsContiguous",
    "tensorLoad", "tensorView", "tensorPermute", "tensorSlice",
    "llaisysAdd", "llaisysArgmax", "llaisysEmbedding", "llaisysLinear", "llaisysRearrange", "llaisysRmsNorm",
    "llaisysROPE", "llaisysSelfAttention", "llaisysSwiGLU",
}


def declared_symbols() -> set[str]:
    names = set()
    for header in INCLUDE.rglob("*.h"):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        text = "\n".join(ln for ln in text.splitlines() if not ln.lstrip().startswith("#"))  # drop macros
        for m in re.finditer(r"LLAISYS_API\s+[^;()]*?\b(\w+)\s*\(", text):
            names.add(m.group(1))
    return names


def test_headers_declare_the_reference_abi():
    assert REFERENCE_SYMBOLS <= declared_symbols()


def test_every_declared_symbol_is_exported_and_bound():
    lib = ctypes.CDLL(str(libllaisys.library_path()))
    declared = declared_symbols()
    assert len(declared) >= len(REFERENCE_SYMBOLS) + 20
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"
        assert name in libllaisys.PROTOTYPES, f"{name} has no ctypes prototype"
    assert set(libllaisys.PROTOTYPES) == declared, "binding and headers name different symbols"


def test_enum_values_match_the_reference_abi():
    # reference: include/llaisys.h:23-64 and python/llaisys/libllaisys/llaisys_types.py:6-47
    assert (llaisys.DeviceType.CPU, llaisys.DeviceType.NVIDIA) == (0, 1)
    assert (llaisys.DataType.I64, llaisys.DataType.F16, llaisys.DataType.F32, llaisys.DataType.BF16) == (6, 12, 13, 19)
    assert [int(k) for k in llaisys.MemcpyKind] == [0, 1, 2, 3]


def test_runtime_table_layout_and_cpu_device():
    api = llaisys.RuntimeAPI(llaisys.DeviceType.CPU)
    assert api.get_device_count() == 1
    assert ctypes.sizeof(libllaisys.LlaisysRuntimeAPI) == 12 * ctypes.sizeof(ctypes.c_void_p)
    # NVIDIA table exists even with no GPU: it reports a count and never crashes the probe
    assert llaisys.RuntimeAPI(llaisys.DeviceType.NVIDIA).get_device_count() >= 0
