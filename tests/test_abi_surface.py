"""The drop-in boundary, checked without a GPU: the shared library loads, exports every symbol the
header declares, the v1 launch order is the reference's, and the ABI description fails closed the
way the reference's does (its tests/test_abi.py, test_launch_signature.py, test_layout_and_scaffold.py)."""
import ctypes
import re
import subprocess
from pathlib import Path

import pytest

from jacq_b200 import _native, abi, bindings
from jacq_b200.layout import KiviModelGeometry, KiviPageLayout

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "jacq_kivi_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.DOTALL)
    names = re.findall(r"^\s*(?:int|void|size_t|const char\*)\s+(\w+)\s*\(", text, flags=re.MULTILINE)
    return sorted(set(names))


def launch_params(symbol):
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.DOTALL)
    m = re.search(r"void\s+" + symbol + r"\s*\((.*?)\);", text, flags=re.DOTALL)
    assert m, symbol
    return [re.findall(r"[A-Za-z_][A-Za-z0-9_]*$", p.strip())[0] for p in m.group(1).split(",")]


def test_header_declares_the_whole_surface():
    names = declared_functions()
    assert set(names) == set(abi.V1_SYMBOLS) | set(abi.V2_SYMBOLS)
    assert set(names) == set(_native.SIGNATURES)


def test_library_loads_and_exports_every_declared_symbol(native_lib):
    for name in declared_functions():
        assert getattr(native_lib, name) is not None, name
    assert native_lib.kivi_b200_abi_version() == abi.JACQ_KIVI_ABI_VERSION == 2
    for code, name in _native.STATUS_NAMES.items():
        assert native_lib.kivi_b200_status_string(code)
    assert native_lib.kivi_b200_status_string(99) == b"unknown status"


def test_library_exports_the_reference_cxx_writer_symbols(native_lib):
    """The reference's binding declares kivi_cache_write_launch / _batched_launch with C++ linkage
    (integrations/vllm_kivi/source_patch.py:624-637); the library must satisfy that link too."""
    out = subprocess.run(["nm", "-D", "--defined-only", "-C", str(_native.LIB_PATH)], capture_output=True, text=True,
                         check=True).stdout
    assert re.search(r"\bkivi_cache_write_launch\(unsigned char\*, __half\*", out)
    assert re.search(r"\bkivi_cache_write_batched_launch\(unsigned char\*, __half\*", out)


def test_jac_launch_order_matches_the_reference_binding():
    emitted = launch_params("jac_launch")
    assert emitted == ["Q", "BLOCK_TABLE", "K_CODE_PAGES", "K_SCALE_PAGES", "K_ZERO_PAGES", "V_CODE_PAGES",
                       "V_SCALE_PAGES", "V_ZERO_PAGES", "K_RESIDUAL_SCRATCH", "V_RESIDUAL_SCRATCH", "SEQ_LEN", "O",
                       "stream"]
    expected = bindings.default_qwen32b_binding_abi().jac_launch_order()
    assert expected[-1] == "cudaStream_t stream"
    assert expected[:-1] == emitted[:-1]
    assert "K_RESIDUAL" not in expected and "V_RESIDUAL" not in expected
    report = abi.kernel_interface()
    decode = [k for k in report["kernels"] if k["torch_op"] == "kivi_decode_dsl"][0]
    assert decode["launch_order"][:-1] == emitted[:-1]
    assert launch_params("jac_launch_tp2_local") == emitted
    assert launch_params("jac_launch_batched")[:3] == ["Q", "SEQ_LENS", "BLOCK_TABLE"]
    assert launch_params("jac_launch_batched")[-3:] == ["NUM_QUERIES", "O", "stream"]
    assert launch_params("jac_launch_sparse_retained")[-4:] == ["SEQ_LEN", "NUM_RETAINED_PAGES", "O", "stream"]
    assert launch_params("jac_launch_cache_write")[-5:] == ["NEW_K", "NEW_V", "BLOCK_TABLE", "SEQ_LEN", "stream"]
    assert launch_params("jac_launch_cache_write_batched")[-4:] == ["BLOCK_TABLE", "START_SEQ_LEN", "NUM_NEW", "stream"]


def test_v1_cap_and_fail_closed_checks():
    assert abi.MAX_SEQ_LEN == 4096 == abi.OLD_BLOCKS_CAP * abi.BLOCK_SIZE + abi.RESIDUAL_TOKENS
    with pytest.raises(abi.UnsupportedAbiError):
        abi.kernel_interface(seq_len=4097)
    report = abi.kernel_interface(seq_len=4096)
    assert report["old_pages"] == 124 and report["seq_len"] == 4096
    assert set(abi.REQUIRED_TORCH_OPS) == {"kivi_decode_dsl", "kivi_cache_write_dsl", "kivi_cache_write_jac_dsl"}
    assert abi.CACHE_WRITE_KERNELS == ("hand_cuda", "jac_dsl")
    for bad in ("0.9.1", "0.8.4", "0.8.50", "0.8.55", "0.8.5.1", "0.8.5x", "0.8.5-rc1+gdeadbeef"):
        with pytest.raises(abi.UnsupportedAbiError):
            abi.check_vllm_version(bad)
    for good in ("0.8.5", "0.8.5.post2", "0.8.5.post2.dev0+g3015d5634.d20260815"):
        abi.check_vllm_version(good)
    abi.check_vllm_version("0.8.5", abi.SUPPORTED_VLLM_SOURCE_HEAD)
    with pytest.raises(abi.UnsupportedAbiError):
        abi.check_vllm_version("0.8.5", "0" * 40)
    abi.check_cuda_arch("sm_100")
    for arch in ("sm_89", "sm_90", "sm_120"):
        with pytest.raises(abi.UnsupportedAbiError):
            abi.check_cuda_arch(arch)
    abi.check_geometry(KiviModelGeometry.qwen25_coder_32b())
    with pytest.raises(abi.UnsupportedAbiError):
        abi.check_geometry(KiviModelGeometry.mistral_7b())


def test_page_byte_accounting_matches_the_reference_goldens():
    lay = KiviPageLayout(KiviModelGeometry.qwen25_coder_32b())
    rep = lay.to_abi_dict(seq_len=4096)
    assert rep["fp16_page_bytes_per_layer"] == 131_072
    assert rep["key_code_bytes"] == rep["value_code_bytes"] == 16_384
    assert rep["key_scale_zero_bytes"] == rep["value_scale_zero_bytes"] == 4_096
    assert rep["quantized_page_bytes_per_layer"] == 40_960
    assert rep["residual_pages"] == 4
    assert rep["effective_bytes_per_token_all_layers_at_seq_len"] == 87_552.0
    assert 2.99 < rep["capacity_ratio_vs_fp16_at_seq_len"] < 3.0
    with pytest.raises(ValueError, match="block_size==group_size"):
        KiviPageLayout(KiviModelGeometry.qwen25_coder_32b(), block_size=16).validate_for_vllm_lane()
    KiviPageLayout(KiviModelGeometry.qwen25_coder_32b(), block_size=16).validate_for_b200_lane()
    with pytest.raises(ValueError):
        KiviPageLayout(KiviModelGeometry.qwen25_coder_32b(), block_size=24).validate_for_b200_lane()


def test_decode_bytes_of_the_benchmark_configs():
    """Algorithmic bytes per decode step (one layer): the roofline denominators."""
    from jacq_b200.cache import model_layout
    assert model_layout("tinyllama").decode_algorithmic_bytes(512) * 4 == 795_104
    assert model_layout("qwen2.5-0.5b").decode_algorithmic_bytes(4096) * 64 == 43_073_024
    assert model_layout("mistral-7b").decode_algorithmic_bytes(8192) * 128 == 1_193_537_536
    assert model_layout("reference-lane").decode_algorithmic_bytes(4096) == 5_634_544


def test_v2_interface_and_host_only_calls(native_lib):
    from jacq_b200.cache import geometry_struct, model_layout
    rep = abi.kernel_interface_v2(model_layout("mistral-7b"), 8192)
    assert rep["max_old_pages"] == 504 and rep["abi_version"] == 2
    names = [b["name"] for b in rep["tensor_bindings"]]
    assert names[2:10] == list(bindings.CACHE_TENSORS)
    scratch = rep["tensor_bindings"][8]
    assert scratch["shape"] == [8, 256, 128]
    for key, fast in [("mistral-7b", 1), ("tinyllama", 1), ("qwen2.5-0.5b", 1), ("reference-lane", 1)]:
        g = geometry_struct(model_layout(key))
        flag = ctypes.c_int(-1)
        assert native_lib.kivi_b200_validate_geometry(ctypes.byref(g), ctypes.byref(flag)) == 0
        assert flag.value == fast
    bad = _native.KiviGeometry(32, 8, 128, 16, 24, 128)     # group not a multiple of block
    assert native_lib.kivi_b200_validate_geometry(ctypes.byref(bad), None) == 2
    odd = _native.KiviGeometry(24, 2, 96, 16, 32, 32)        # head_dim 96, 12 heads per group: generic kernel
    flag = ctypes.c_int(-1)
    assert native_lib.kivi_b200_validate_geometry(ctypes.byref(odd), ctypes.byref(flag)) == 0 and flag.value == 0
    g = geometry_struct(model_layout("mistral-7b"))
    assert native_lib.kivi_b200_decode_workspace_bytes(ctypes.byref(g), 128, 8192) >= 256   # unsplit plan: a token amount
    assert native_lib.kivi_b200_decode_workspace_bytes(ctypes.byref(g), 1, 32768) > 8 * 8 * 4 * 130 * 4
    assert native_lib.kivi_b200_decode_workspace_bytes(ctypes.byref(bad), 1, 100) == 0
    # argument validation happens on the host, before anything is launched
    assert native_lib.kivi_b200_gemv_f16(None, None, None, None, 8, 8, 1, None) == 1
    assert native_lib.kivi_b200_decode(ctypes.byref(g), None, None, None, 0, None, None, 1, 1, None, None, 0, None) == 1


def test_v1_writer_symbols_refuse_a_non_positive_head_count(native_lib):
    """NKV_RUNTIME <= 0 is refused with a message and exit(1) before anything is computed from it (the reference
    would report an invalid launch configuration, integrations/vllm_kivi/source_patch.py:1661-1697). Run in a
    child process, since the v1 contract is print-and-exit; no GPU is touched."""
    import sys
    code = (
        "import ctypes, sys\n"
        f"lib = ctypes.CDLL({str(_native.LIB_PATH)!r})\n"
        "null = ctypes.c_void_p(0)\n"
        "args = [null] * 12 + [ctypes.c_int(200), ctypes.c_int(int(sys.argv[1])), null]\n"
        "lib.kivi_b200_cache_write_launch(*args)\n"
        "print('returned')\n")
    for nkv in (0, -3):
        proc = subprocess.run([sys.executable, "-c", code, str(nkv)], capture_output=True, text=True, timeout=120)
        assert proc.returncode == 1, (proc.returncode, proc.stdout, proc.stderr)
        assert "NKV_RUNTIME out of range" in proc.stderr and "returned" not in proc.stdout
