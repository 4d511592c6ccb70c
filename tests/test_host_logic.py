"""Host-side logic of the v1 adapter and the sharding helpers, on CPU tensors: every check the
reference's backend stub makes (integrations/vllm_kivi/source_patch.py:179-553) fires with the
same exception type before any library call."""
from pathlib import Path
import pytest
import torch

from jacq_b200 import kivi_dsl, sharding


def cpu_bundle(nkv=8, nb=4):
    return {
        "kind": kivi_dsl.KIVI_CACHE_KIND, "jac_launch_order": kivi_dsl.JAC_LAUNCH_ORDER,
        "K_CODE_PAGES": torch.zeros((nb, nkv, 32, 64), dtype=torch.uint8),
        "K_SCALE_PAGES": torch.zeros((nb, nkv, 128), dtype=torch.float16),
        "K_ZERO_PAGES": torch.zeros((nb, nkv, 128), dtype=torch.float16),
        "V_CODE_PAGES": torch.zeros((nb, nkv, 32, 64), dtype=torch.uint8),
        "V_SCALE_PAGES": torch.zeros((nb, nkv, 32, 4), dtype=torch.float16),
        "V_ZERO_PAGES": torch.zeros((nb, nkv, 32, 4), dtype=torch.float16),
        "K_RESIDUAL_SCRATCH": torch.zeros((nkv, 160, 128), dtype=torch.float16),
        "V_RESIDUAL_SCRATCH": torch.zeros((nkv, 160, 128), dtype=torch.float16),
    }


def test_cache_bundle_validation():
    b = cpu_bundle()
    kivi_dsl.validate_kivi_cache_bundle(b)
    with pytest.raises(TypeError):
        kivi_dsl.validate_kivi_cache_bundle({**b, "kind": "other"})
    with pytest.raises(KeyError):
        kivi_dsl.validate_kivi_cache_bundle({k: v for k, v in b.items() if k != "V_ZERO_PAGES"})
    with pytest.raises(TypeError):
        kivi_dsl.validate_kivi_cache_bundle({**b, "K_CODE_PAGES": b["K_CODE_PAGES"].to(torch.int8)})
    with pytest.raises(TypeError):
        kivi_dsl.validate_kivi_cache_bundle({**b, "K_RESIDUAL_SCRATCH": b["K_RESIDUAL_SCRATCH"].float()})


def test_decode_binding_checks_fire_in_the_reference_order():
    b = cpu_bundle()
    q = torch.zeros((40, 128), dtype=torch.float16)
    o = torch.zeros((40, 128), dtype=torch.float32)
    bt = torch.zeros(124, dtype=torch.int32)
    mk = lambda **kw: kivi_dsl.KiviDslLaunchBinding(kw.get("q", q), kw.get("bt", bt), kw.get("cache", b),
                                                    kw.get("seq_len", 100), kw.get("out", o)).jac_launch_args()
    assert mk()[-2:] == (100, o)
    with pytest.raises(RuntimeError):
        mk(cache={**b, "jac_launch_order": ("Q",)})
    with pytest.raises(TypeError):
        mk(bt=bt.long())
    with pytest.raises(TypeError):
        mk(q=q.float())
    with pytest.raises(TypeError):
        mk(out=o.half())
    for bad in (0, 4097):
        with pytest.raises(ValueError):
            mk(seq_len=bad)
    # CPU tensors pass the dtype checks and are then refused: there is no CPU path
    with pytest.raises(RuntimeError):
        kivi_dsl.launch_kivi_dsl_decode(q, bt, b, o, seq_len=100)


@pytest.mark.parametrize("seq_len,required", [(128, 0), (129, 0), (159, 0), (160, 1), (191, 1), (192, 2), (4096, 124)])
def test_block_table_width_guard(seq_len, required):
    """Boundary table of the reference's C++ guard test (tests/test_runtime_guards.py:163-165)."""
    kivi_dsl._check_block_table_width(torch.zeros(max(required, 0), dtype=torch.int32), seq_len)
    if required > 0:
        with pytest.raises(RuntimeError):
            kivi_dsl._check_block_table_width(torch.zeros(required - 1, dtype=torch.int32), seq_len)
    for invalid in (0, 4097):
        with pytest.raises(ValueError):
            kivi_dsl._check_block_table_width(torch.zeros(124, dtype=torch.int32), invalid)


def test_writer_argument_checks():
    b = cpu_bundle()
    k = torch.zeros((8, 128), dtype=torch.float16)
    sm = torch.zeros(1, dtype=torch.int64)
    bt = torch.zeros(124, dtype=torch.int32)
    with pytest.raises(TypeError):
        kivi_dsl.require_kivi_cache_write(k.float(), k, sm, bt, b, 1)
    with pytest.raises(TypeError):
        kivi_dsl.require_kivi_cache_write(k, k, sm.int(), bt, b, 1)
    with pytest.raises(TypeError):
        kivi_dsl.require_kivi_cache_write(k, k, sm, bt.long(), b, 1)
    with pytest.raises(RuntimeError):
        kivi_dsl.require_kivi_cache_write(k[:4], k, sm, bt, b, 1)
    with pytest.raises(RuntimeError):   # all checks passed, tensors are not on a GPU
        kivi_dsl.require_kivi_cache_write(k, k, sm, bt, b, 1)
    for n in (0, 161):
        with pytest.raises(ValueError):
            kivi_dsl.require_kivi_cache_write_batched(k, k, sm, bt, b, 0, n)
    with pytest.raises(ValueError):
        kivi_dsl.require_kivi_cache_write_batched(torch.zeros((10, 8, 128), dtype=torch.float16),
                                                  torch.zeros((10, 8, 128), dtype=torch.float16), sm, bt, b, 4090, 10)


def test_batched_and_sparse_decode_checks():
    b = cpu_bundle()
    q = torch.zeros((3, 40, 128), dtype=torch.float16)
    o = torch.zeros((3, 40, 128), dtype=torch.float32)
    bt = torch.zeros(124, dtype=torch.int32)
    lens = torch.tensor([1, 4096, 4097], dtype=torch.int32)
    with pytest.raises(ValueError, match=r"SEQ_LENS\[2\]"):
        kivi_dsl.launch_kivi_dsl_decode_batched(q, lens, bt, b, o, num_queries=3)
    with pytest.raises(TypeError):
        kivi_dsl.launch_kivi_dsl_decode_batched(q, lens.long(), bt, b, o, num_queries=3)
    with pytest.raises(ValueError):
        kivi_dsl.launch_kivi_dsl_decode_batched(q, lens, bt, b, o, num_queries=161)
    with pytest.raises(ValueError):
        kivi_dsl.launch_kivi_dsl_decode_sparse_retained(q[0], bt[:100], b, o[0], seq_len=500, num_retained_pages=3)
    with pytest.raises(ValueError):
        kivi_dsl.launch_kivi_dsl_decode_sparse_retained(q[0], bt, b, o[0], seq_len=500, num_retained_pages=125)


def test_cache_write_kernel_selector(monkeypatch):
    monkeypatch.delenv(kivi_dsl.CACHE_WRITE_KERNEL_ENV, raising=False)
    assert kivi_dsl.cache_write_kernel_source() == "hand_cuda"
    for raw, want in [("jac-dsl", "jac_dsl"), (" DSL ", "jac_dsl"), ("legacy", "hand_cuda"), ("CUDA", "hand_cuda")]:
        monkeypatch.setenv(kivi_dsl.CACHE_WRITE_KERNEL_ENV, raw)
        assert kivi_dsl.cache_write_kernel_source() == want
    monkeypatch.setenv(kivi_dsl.CACHE_WRITE_KERNEL_ENV, "fastest")
    with pytest.raises(ValueError):
        kivi_dsl.cache_write_kernel_source()


def test_plan_batched_write_invariants():
    for start, n in [(0, 1), (0, 512), (127, 34), (159, 1), (160, 400), (4000, 96)]:
        pieces = kivi_dsl.plan_batched_write(start, n)
        assert pieces[0].start_seq_len == start and sum(p.num_new for p in pieces) == n
        seq = start
        for p in pieces:
            assert p.start_seq_len == seq and 1 <= p.num_new <= 160
            old0 = max(0, seq - 128) // 32 * 32
            old1 = max(0, seq + p.num_new - 128) // 32 * 32
            assert old1 - old0 in (0, 32)
            assert p.scratch_start == seq - old0
            assert (p.age_out_page is None) == (old1 == old0)
            if old1 > old0:
                assert p.age_out_page == old0 // 32 and p.post_shift_residual_len == seq + p.num_new - old1
            seq += p.num_new
    with pytest.raises(ValueError):
        kivi_dsl.plan_batched_write(-1, 1)
    with pytest.raises(ValueError):
        kivi_dsl.plan_batched_write(0, 0)


def test_sharding_helpers():
    shards = sharding.contiguous_shards(10, 4)
    assert [list(s) for s in shards] == [[0, 1, 2], [3, 4, 5], [6, 7], [8, 9]]
    costs = [32768, 1, 20000, 5, 16000, 16000, 9000, 7]
    b = sharding.balanced_shards(costs, 2)
    assert sorted(b[0] + b[1]) == list(range(8))
    assert sharding.shard_imbalance(costs, b) < 1.05
    assert sharding.shard_imbalance(costs, [list(r) for r in sharding.contiguous_shards(8, 2)]) > 1.1
    assert sharding.balanced_shards([], 3) == [[], [], []]


def test_retained_tables_compaction_on_cpu():
    """Compact tables and counts of the sparse-retained decode: kept pages first in their original
    order, the count is the kept pages among the dense old pages of the current length."""
    import torch
    from jacq_b200.cache import KiviCache, model_layout
    cache = KiviCache.__new__(KiviCache)          # the arithmetic needs no device
    cache.layout = model_layout("reference-lane")  # block = group = 32, residual 128
    cache.device = torch.device("cpu")
    tables = torch.arange(100, 110, dtype=torch.int32).repeat(3, 1) + torch.tensor([[0], [1000], [2000]], dtype=torch.int32)
    mask = torch.ones((3, 10), dtype=torch.bool)
    mask[0, [1, 3]] = False                         # sequence 0 dropped pages 1 and 3
    mask[2, :4] = False                             # sequence 2 dropped its first four pages
    lens = torch.tensor([128 + 6 * 32 + 5, 128 + 2 * 32, 128 + 5 * 32 + 31], dtype=torch.int32)   # 6, 2, 5 dense old pages
    compact, counts = cache.retained_tables(lens, tables, mask)
    assert counts.tolist() == [4, 2, 1]
    assert compact[0, :4].tolist() == [100, 102, 104, 105]
    assert compact[1, :2].tolist() == [1100, 1101]
    assert compact[2, :1].tolist() == [2104]
    assert sorted(compact[0].tolist()) == sorted(tables[0].tolist())   # a permutation: nothing lost


def test_library_artifact_places_forwarding_units(tmp_path, native_lib):
    """The vLLM-lane artefact for the prebuilt library: every kernel file of the reference's flow
    gets a unit that defines nothing, the header and a CMake fragment ride along."""
    from jacq_b200 import abi, dsl_decode
    root = Path(__file__).resolve().parent.parent
    art = dsl_decode.B200KernelLibraryArtifact(str(root), str(tmp_path))
    rep = art.report()
    assert rep["library_exists"] and rep["header_exists"] and rep["abi_version"] == abi.JACQ_KIVI_ABI_VERSION
    assert set(rep["symbols"]) <= set(abi.V1_SYMBOLS) | {"kivi_cache_write_launch", "kivi_cache_write_batched_launch"}
    assert not any(rep["kernel_files"].values())
    written = art.emit()
    assert all(p.exists() for p in written)
    unit = (tmp_path / "csrc/kivi/decode_attention_kivi_batched_dsl.cu").read_text()
    assert "Library artifact for embedding in a runtime extension" in unit and "jac_launch_batched" in unit
    assert "__global__" not in unit and "int main(" not in unit and 'extern "C" void' not in unit
    assert (tmp_path / "csrc/kivi/jacq_kivi_b200.h").read_text() == (root / "include/jacq_kivi_b200.h").read_text()
    cmake = (tmp_path / "csrc/kivi/jacq_kivi_b200.cmake").read_text()
    assert "IMPORTED_LOCATION" in cmake and "libjacq_kivi_b200.so" in cmake
    rep = art.report()
    assert all(rep["kernel_files"].values())
    assert rep["serving_env"]["JAC_VLLM_KIVI_DECODE_KERNEL_SOURCE"] == "b200-kivi-library"
