"""CPU-only checks of the boundary: the library loads, exports every declared symbol, and rejects bad calls on the
host before anything would be launched. No compute call is made here."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def L():
    from pragnosia_b200 import build, _lib
    build.build()
    return _lib.lib()


def declared_symbols():
    text = (ROOT / "include" / "pragnosia_b200.h").read_text()
    return sorted(set(re.findall(r"^(?:int|long long|const char \*)\s*(pgb_[a-z0-9_]+)\(", text, flags=re.M)))


def test_every_declared_symbol_is_exported(L):
    names = declared_symbols()
    assert len(names) >= 9
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/pragnosia_b200.h but not exported"


def test_binding_table_matches_header(L):
    from pragnosia_b200 import _lib
    header = set(declared_symbols()) - {"pgb_status_string", "pgb_last_cuda_error"}
    assert set(_lib.SIGNATURES) == header


def test_status_strings(L):
    assert L.pgb_abi_version() == 1
    assert L.pgb_status_string(0) == b"ok"
    assert b"NULL" in L.pgb_status_string(1)


def test_bad_calls_are_rejected_on_the_host(L):
    one = ctypes.c_void_p(0x1000)        # a non-null, 16-byte aligned, never dereferenced address
    odd = ctypes.c_void_p(0x1004)
    # null pointers
    assert L.pgb_lambda_scan_fwd(None, one, one, 0, 0, None, None, one, one, one, 1, 1, 4, None) == 1
    # state given only half
    assert L.pgb_lambda_scan_fwd(one, one, one, 0, 0, one, None, one, one, one, 1, 1, 4, None) == 1
    # bad shape
    assert L.pgb_lambda_scan_fwd(one, one, one, 0, 0, None, None, one, one, one, 0, 1, 4, None) == 2
    assert L.pgb_lambda_scan_fwd_ex(one, one, one, 0, 0, None, None, one, one, one, 1, 1, 4, 3, None) == 2
    # unsupported head dim, dtype, precision, alignment in the prefill
    args = lambda D=64, dt=0, prec=0, q=one: (q, one, one, dt, one, None, None, None, None, 0.0, one, dt, one, None, 1, 1, 8, D, prec, None)
    assert L.pgb_aspin_prefill_fwd(*args(D=96)) == 3
    assert L.pgb_aspin_prefill_fwd(*args(dt=7)) == 5
    assert L.pgb_aspin_prefill_fwd(*args(prec=9)) == 2
    assert L.pgb_aspin_prefill_fwd(*args(q=odd)) == 4
    # prep: stride that breaks the per-lane vector alignment
    assert L.pgb_aspin_prep_fwd(one, one, one, 0, 7, 7, 7, None, 0, 0, one, one, one, one, one, 1, 1, 4, 2, 64, None) == 4
    assert L.pgb_aspin_prep_fwd(one, one, one, 0, 512, 128, 64, None, 0, 0, one, one, one, one, one, 1, 1, 4, 2, 32, None) == 3
    # decode: the delta rule without beta; batch stride smaller than a row
    dec = lambda gate=None, delta=0, sb=64: (one, one, one, 0, sb, 1, gate, 1, 1, delta, one, 1, None, one, None, 0.0, one, one,
                                             None, 0.0, one, 0, 64, 1, 1, 64, None)
    assert L.pgb_aspin_decode_step(*dec(delta=1)) == 1
    assert L.pgb_aspin_decode_step(*dec(sb=8)) == 2
    assert L.pgb_rotate_pairs(one, 0, one, one, one, 1, 1, 1, 7, None) == 2
    # fused small-batch linear: norm without its weight, more than eight rows, K not a multiple of 8, unaligned W
    sk = lambda nw=None, kind=0, B=1, K=768, W=one: (one, None, nw, None, kind, 1e-5, W, None, 0, one, None, B, K, 16, None)
    assert L.pgb_skinny_linear(*sk(kind=1)) == 1
    assert L.pgb_skinny_linear(*sk(B=9)) == 7
    assert L.pgb_skinny_linear(*sk(K=100)) == 2
    assert L.pgb_skinny_linear(*sk(W=odd)) == 4
    # decode-step ends: d not a multiple of 8; a negative temperature; a missing ticket
    assert L.pgb_decode_embed(one, one, one, one, one, 1, 60, 10, 10, None) == 2
    assert L.pgb_decode_sample(one, 0, -1.0, 0, one, None, 0, one, None, None, one, 1, 8, 1, None) == 2
    assert L.pgb_decode_sample(one, 0, 1.0, 0, one, None, 0, one, None, None, None, 1, 8, 1, None) == 1


def test_ops_refuse_cpu_tensors():
    from pragnosia_b200 import ops
    x = torch.zeros(1, 4, 8)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.lambda_scan(x, x, x)
    q = torch.zeros(1, 1, 8, 64)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.prefill(q, q, q, torch.zeros(1, 1, 8))


def test_model_loads_reference_named_checkpoints():
    """The modules keep the reference's parameter names and shapes, so its state_dicts load strictly."""
    import oracle
    from pragnosia_b200.model import LM
    for mixer, norm in (("aspin", "ln"), ("dspin", "rms"), ("hspin", "ln"), ("hdspin", "rms"), ("fspin", "ln")):
        cfg = oracle.lm_config(256, 128, 2, 2, 32, mixer, norm)
        m = LM(256, 128, 2, 2, 32, mixer, norm)
        m.load_state_dict(oracle.init_lm_params(cfg, 0), strict=True)
    n = sum(p.numel() for p in LM().parameters())
    assert abs(n / 1e6 - 91.93) < 0.01
    with pytest.raises(NotImplementedError):
        LM(mixer="attn")


def test_lambda_scan_segment_choice(L):
    """The host picks more time segments when there are few channels and never more than the sequence has pieces."""
    ts = lambda B, T, D: L.pgb_lambda_scan_time_segments(B, T, D, 148)
    assert ts(64, 32768, 768) == 8                             # 12288 channel quads x 8 segments: whole rounds of resident warps
    assert ts(1, 32768, 64) == 32                              # 16 quads: the time axis must supply the parallelism
    assert ts(1, 32768, 64) >= ts(8, 32768, 768) >= ts(64, 32768, 768)
    assert ts(2, 1, 300) == 1 and ts(2, 6, 300) <= 2           # a short sequence has nothing to split
    for B, T, D in ((2, 45, 300), (16, 512, 704), (3, 1000, 24)):
        t = ts(B, T, D)
        assert t in (1, 2, 4, 8, 16, 32)
    assert ts(0, 5, 5) == 0 and L.pgb_lambda_scan_time_segments(1, 5, 5, 0) == 0


def test_new_entry_points_reject_bad_calls(L):
    one = ctypes.c_void_p(0x1000)
    assert L.pgb_assoc_out_fwd(one, one, one, 0, one, None, one, 1, 1, 8, 64, None) == 1
    assert L.pgb_assoc_out_fwd(one, one, one, 0, one, one, one, 1, 1, 8, 96, None) == 3
    assert L.pgb_prefix_scan_fwd(one, one, 9, one, one, None, one, one, 1, 1, 1, 64, None) == 5
    assert L.pgb_delta_inv_fwd(ctypes.c_void_p(0x1004), one, one, one, 1, 1, 8, 64, None) == 4
    assert L.pgb_delta_loop_fwd(one, one, 0, one, None, one, None, one, one, one, 1, 1, 8, 64, None) == 1
    assert L.pgb_key_topk_mask(one, 0, 64, 64, 64, 1, 1, 1, 64, 0, None) == 2
    assert L.pgb_key_topk_mask(one, 0, 64, 64, 64, 1, 1, 1, 64, 65, None) == 2
    assert L.pgb_short_conv_fwd(one, 0, 8, 8, one, one, one, one, 1, 1, 8, 4, None) == 2       # cache_in == cache_out
    assert L.pgb_lambda_scan_bwd(one, one, one, one, 0, 0, one, None, None, one, one, one, None, None, 1, 1, 4, None) == 1
    assert L.pgb_lambda_scan_bwd(one, one, one, one, 0, 0, one, one, None, one, one, one, one, None, 1, 1, 4, None) == 1
    assert L.pgb_aspin_prep_bwd(one, one, one, 0, 64, 64, 64, one, 1, 1, one, one, one, one, one, 0, one, one, one, None, one,
                                1, 1, 1, 64, None) == 1                                          # a gate without room for its gradient
    assert L.pgb_decode_sample_ex(one, 0, 1.0, 1.5, 0, one, None, 0, one, None, None, one, 1, 8, 1, None) == 2
    assert L.pgb_skinny_linear_ex(one, None, None, None, 0, 1e-5, one, None, 0, one, None, 1, 768, 16, 4, None) == 2
    assert L.pgb_aspin_prep_bwd_tiles(17) == 3
    # the plain rule's two backward kernels, the batch linear layer
    assert L.pgb_assoc_out_bwd(one, one, one, 0, one, one, one, one, one, one, one, None, 1, 1, 8, 64, None) == 1
    assert L.pgb_assoc_out_bwd(one, one, one, 0, one, one, one, one, one, one, one, one, 1, 1, 8, 96, None) == 3
    assert L.pgb_prefix_scan_bwd(one, one, 7, one, one, one, None, None, one, one, one, one, None, 1, 1, 1, 64, None) == 5
    assert L.pgb_batch_linear(one, one, None, one, 129, 16, 64, 0, None) == 7 and L.pgb_batch_linear(one, one, None, one, 4, 12, 64, 0, None) == 2
    assert L.pgb_batch_linear_ex(one, one, one, one, 4, 16, 64, 0, one, 1, one, one, 1, 1e-5, None, None, 0, None) == 1   # folded norm + bias
    assert L.pgb_batch_linear_ex(one, one, None, one, 4, 16, 64, 0, None, 0, None, None, 0, 0.0, None, None, 2, None) == 2  # unknown flag
    assert L.pgb_batch_linear_parts(768) == 48
    assert L.pgb_decode_set_variant(3) == 2 and L.pgb_decode_set_variant(0) == 0
    assert L.pgb_linear_act_set_variant(6) == 2 and L.pgb_linear_act_set_variant(-1) == 2 and L.pgb_linear_act_set_variant(0) == 0
    # the one-launch decode step: scratch size, then the rejects (bias missing for a layer norm, short scratch, batch, head dim)
    assert L.pgb_decode_token_work_bytes(1, 768, 2328, 3072) == 2 * (4 * 768 + 2328 + 3072)
    tok = lambda **kw: L.pgb_decode_token_fwd(one, 12, one, one, one, kw.get("nb", one), 2, 1e-5, one, one, one, one, kw.get("wb", 10 ** 6),
                                              one, one, kw.get("B", 1), 768, 12, kw.get("D", 64), 2328, 3072, 50257, 512, 0, None)
    assert tok(nb=None) == 1 and tok(wb=10) == 2 and tok(B=5) == 7 and tok(D=96) == 3


def test_bench_table_names_are_kernel_bench_cases():
    """bench.py's per-kernel table is built from kernel_bench cases by name: every name it asks for exists."""
    import ast
    import pathlib
    from pragnosia_b200 import kernel_bench as kb
    src = (pathlib.Path(__file__).resolve().parents[1] / "bench.py").read_text()
    fn = next(n for n in ast.walk(ast.parse(src)) if isinstance(n, ast.FunctionDef) and n.name == "kernel_rooflines")
    names = [c.value for t in ast.walk(fn) if isinstance(t, ast.Tuple) for c in t.elts if isinstance(c, ast.Constant) and isinstance(c.value, str)]
    asked = [n for n in names if n in kb.CASES or n.startswith(("prefill", "decode", "lambda", "layer_"))]
    assert len(asked) >= 15 and all(n in kb.CASES for n in asked), [n for n in asked if n not in kb.CASES]
    assert all(n in kb.CASES for n in kb.FLOPS)
