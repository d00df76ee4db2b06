"""CPU: the C-ABI library is built, loads, and exports every symbol include/hilda_b200.h declares;
the ctypes signature table covers the same set. No compute call is made (no GPU here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    src = open(os.path.join(ROOT, "include", "hilda_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(hilda_[a-z0-9_]+)\s*\(", src)))


@pytest.fixture(scope="module")
def libpath():
    from hilda_kernel_b200 import _build
    return _build.build()


def test_header_symbols_exported(libpath):
    lib = ctypes.CDLL(libpath)
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/hilda_b200.h but not exported"


def test_signature_table_matches_header(libpath):
    from hilda_kernel_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared()
    assert _lib.lib() is not None  # binds every signature


def test_size_queries_need_no_gpu(libpath):
    from hilda_kernel_b200 import _lib
    lib = _lib.lib()
    assert lib.hilda_flce_logits_pitch(128256) == 128256
    assert lib.hilda_flce_logits_pitch(16032) == 16128
    assert lib.hilda_flce_padded_rows(100) == 256
    assert lib.hilda_flce_stat_tiles(128256) == 501
    default = lib.hilda_gemm_get_pair()
    try:
        lib.hilda_gemm_set_pair(0)
        assert lib.hilda_flce_default_chunk_rows(16384, 4096, 128256) == 4736  # 37 x 16 tiles = 4 waves of 148 SMs
        lib.hilda_gemm_set_pair(7)
        assert lib.hilda_flce_default_chunk_rows(16384, 4096, 128256) == 4608  # 18 x 16 pair tiles <= 4 waves of 74
    finally:
        lib.hilda_gemm_set_pair(default)
    assert lib.hilda_flce_default_chunk_rows(100, 64, 1000) == 100
    assert lib.hilda_flce_default_chunk_rows(4096, 4096, 128256) == 4096
    one = lib.hilda_flce_workspace_bytes(4096, 4096, 128256, 4096, 1, 0)
    four = lib.hilda_flce_workspace_bytes(16384, 4096, 128256, 4096, 1, 0)
    assert four - one >= 128256 * 4096 * 4  # the fp32 dW accumulator appears only with > 1 chunk
    # compaction on the device adds the index lists and the compacted hidden / d(hidden) copies
    compact = lib.hilda_flce_workspace_bytes(16384, 4096, 128256, 4096, 1, 1)
    assert compact - four >= 2 * 16384 * 4096 * 2 + 16384 * 20
    assert lib.hilda_cross_entropy_workspace_bytes(8192) >= 16
    assert lib.hilda_grpo_workspace_bytes(16) >= 16 + 64


def test_no_cpu_fallback():
    import torch
    import hilda_kernel_b200 as hk
    x = torch.randn(4, 64)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        hk.hilda_rms_norm(x, torch.ones(64))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        hk.hilda_swiglu(x, x)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        hk.hilda_cross_entropy(x, torch.zeros(4, dtype=torch.long))


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "hilda_kernel_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text, f"{f} mentions the oracle"


def test_exported_names_match_reference_api():
    import hilda_kernel_b200 as hk
    for name in ["HildaRMSNormFunction", "hilda_rms_norm", "RMSNorm", "HildaRopeFunction", "hilda_rope",
                 "RotaryEmbedding", "HildaCrossEntropyFunction", "hilda_cross_entropy", "CrossEntropyLoss",
                 "HildaSwiGLUFunction", "hilda_swiglu", "SwiGLU", "HildaGeGLUFunction", "hilda_geglu", "GeGLU",
                 "HildaFusedAddRMSNormFunction",
                 "hilda_fused_add_rms_norm", "FusedAddRMSNorm", "HildaFusedLinearCrossEntropyFunction",
                 "hilda_fused_linear_cross_entropy", "FusedLinearCrossEntropyLoss", "HildaGRPOLossFunction",
                 "hilda_grpo_loss", "GRPOLoss", "fused_selective_log_softmax"]:
        assert hasattr(hk, name), name
    from hilda_kernel_b200.kernels.rope import rope_backward, rope_forward  # used by bench_rope.py:19
    import inspect
    sig = inspect.signature(hk.hilda_grpo_loss)
    assert list(sig.parameters) == ["logits", "completion_ids", "advantages", "old_logp", "ref_logp",
                                    "completion_mask", "temperature", "beta", "eps_low", "eps_high"]
    assert inspect.signature(hk.RMSNorm.__init__).parameters["hidden_dim"] is not None


def test_kernel_choice_setters_and_split_plan_without_a_gpu():
    """The kernel-choice setters round-trip (tensor-core kernels are the default) and the paged
    attention workspace covers one partial result (m, l, 128 sums) per sequence, head and context
    slice of the plan; host-side arithmetic only, no launch."""
    import hilda_kernel_b200._lib as L
    lib = L.lib()
    for setter in (lib.hilda_attn_res_set_path,):
        assert setter(-1) == 1          # out of range: unchanged, returns the current choice
        assert setter(0) == 1 and setter(-1) == 0
        assert setter(1) == 0 and setter(-1) == 1
    part = (128 + 2) * 4
    big = lib.hilda_paged_attention_fp8_workspace_bytes(32, 16, 8, 16, 256)
    assert (big - 256) % (32 * 16 * part) == 0 and 2 <= (big - 256) // (32 * 16 * part) <= 64
    assert lib.hilda_paged_attention_fp8_workspace_bytes(4096, 16, 8, 1, 16) == 256   # one slice: no partials
    assert lib.hilda_paged_attention_fp8_workspace_bytes(0, 16, 8, 16, 256) == 256


def test_row_engine_plan_covers_every_vocabulary_and_is_instantiated():
    """Host-side only: for every vocabulary size in a dense sweep (and the published ones) the plan of the
    CrossEntropy / GRPO row engine holds the whole row (threads x vectors per thread x cluster >= the row's
    vectors), stays within the portable cluster size, and names a kernel the library was built with."""
    import ctypes
    import hilda_kernel_b200._lib as L
    lib = L.lib()
    out = (ctypes.c_int * 4)()
    named = [32000, 32001, 32768, 49152, 50257, 50304, 65536, 100352, 102400, 128256, 129280, 151643, 151936, 152064,
             200064, 201088, 256000, 262144]
    sizes = sorted(set(named) | set(range(8, 4096, 7)) | set(range(4096, 330000, 509)))
    for dtype, vec, limit in ((0, 4, 8 * 512 * 19 * 4), (1, 8, 8 * 512 * 19 * 8), (2, 8, 8 * 512 * 19 * 8)):
        for v in sizes:
            vector = lib.hilda_row_engine_plan(v, dtype, out)
            th, nv, cl, ns = out[0], out[1], out[2], out[3]
            if not vector:
                assert v < 4 * vec or v // vec > limit // vec, (v, dtype)   # only tiny or huge rows take the scalar kernel
                continue
            assert cl in (1, 2, 4, 8) and th in (256, 512)
            # the vectors are the aligned body of the row; up to vec - 1 elements before and after it are scalars
            assert (nv + ns) * cl * th >= v // vec, (v, dtype, th, nv, cl, ns)
            assert ns * th * 16 <= 100 * 1024
            assert lib.hilda_row_engine_has_kernel(th, nv, cl, ns) == 1, (v, dtype, th, nv, cl, ns)
    assert lib.hilda_row_engine_has_kernel(256, 8, 4, 5) == 0


def test_top_level_kernels_package_like_the_reference_benches():
    """hilda-kernel's bench scripts put their package's parent directory first on sys.path and import
    ``kernels.<op>`` (benchmarks/bench_rms_norm.py:17-19, bench_rope.py:19, bench_grpo.py:6-8). With
    ``hilda_kernel_b200/`` in that place the same statements must resolve to this library, from a
    working directory that is not the repository, in a fresh interpreter."""
    import subprocess
    import sys
    import tempfile
    code = (
        "import sys\n"
        f"sys.path.insert(0, {os.path.join(ROOT, 'hilda_kernel_b200')!r})\n"
        "from kernels.rms_norm import hilda_rms_norm, RMSNorm\n"
        "from kernels.fused_add_rms_norm import hilda_fused_add_rms_norm\n"
        "from kernels.rope import hilda_rope, rope_forward, rope_backward\n"
        "from kernels.swiglu import hilda_swiglu\n"
        "from kernels.cross_entropy import hilda_cross_entropy\n"
        "from kernels.fused_linear_cross_entropy import hilda_fused_linear_cross_entropy\n"
        "from kernels.grpo_loss import hilda_grpo_loss, fused_selective_log_softmax\n"
        "from kernels import RMSNorm as R2, FusedLinearCrossEntropyLoss, GRPOLoss\n"
        "import kernels, hilda_kernel_b200.kernels.rms_norm as real\n"
        "assert kernels.rms_norm is real and RMSNorm is real.RMSNorm is R2\n"
        "assert RMSNorm(8).weight.shape == (8,)\n"
        "print('dropin ok')\n")
    env = {k: v for k, v in os.environ.items() if k != "PYTHONPATH"}
    with tempfile.TemporaryDirectory() as tmp:
        r = subprocess.run([sys.executable, "-c", code], cwd=tmp, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "dropin ok" in r.stdout, r.stderr[-2000:]


def test_debug_flag_compiles(tmp_path):
    """The -DHILDA_DEBUG variant (every launch followed by a synchronise-and-check) compiles for
    sm_100a; two small sources stand for the whole library here, the full debug build takes minutes."""
    import subprocess
    from hilda_kernel_b200 import _build
    for name in ("swiglu.cu", "rope.cu"):
        obj = str(tmp_path / (name + ".o"))
        cmd = _build.compile_one(os.path.join(_build.CSRC, name), obj, debug=True)
        assert "-DHILDA_DEBUG" in cmd
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0 and os.path.getsize(obj) > 0, r.stderr[-2000:]


def test_bench_reference_arm_prints_the_contract_line(tmp_path):
    """`bench.py --impl reference` runs the CPU restatement of the reference on a row sample of the
    same workload and prints ONE JSON line whose metric, unit and config.workload are the ones the
    GPU arm prints (a small shape here, so that it takes seconds)."""
    import json
    import subprocess
    import sys
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                        "--bt", "256", "--vocab", "4096", "--hidden", "256"], capture_output=True, text=True, timeout=600,
                       cwd=str(tmp_path))
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip().startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "FusedLinearCE fwd+bwd tokens/s" and d["unit"] == "tokens/s"
    assert d["higher_is_better"] is True and d["value"] > 0 and d["vs_baseline"] is None
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    sys.path.insert(0, ROOT)
    import bench
    bench.BT, bench.V, bench.H = 256, 4096, 256
    try:
        assert d["config"]["workload"] == bench.workload_name()
        t = bench.make_targets()
        assert t.shape == (256,) and int((t == -100).sum()) == round(0.05 * 256)
    finally:
        bench.BT, bench.H, bench.V = 16384, 4096, 128256
