"""The decode step as ONE launch per token (decode_token.cu) against the same step chained from this library's separate
kernels (five launches a layer), whose parity with the oracle the model tests pin: same roundings, same accumulation
order, so logits and states are compared at a few bf16 ulps, ids exactly."""
import pytest
import torch

from pragnosia_b200 import _lib, synth
from pragnosia_b200.generate import Decoder

from test_gpu_model import DEV, close, small_lm

pytestmark = pytest.mark.gpu


def healthy():
    import ctypes
    flag = ctypes.c_int(-1)
    assert _lib.lib().pgb_tc_error_flag(ctypes.byref(flag)) == 0
    return flag.value


@pytest.mark.parametrize("mixer,norm", [("aspin", "rms"), ("aspin", "ln"), ("dspin", "ln"), ("hspin", "rms"), ("hdspin", "ln")])
@pytest.mark.parametrize("B", [1, 2, 3, 4])
def test_one_launch_step_matches_the_chained_kernels(mixer, norm, B):
    m, _, _ = small_lm(mixer, norm, torch.bfloat16)
    ids = synth.token_ids(B, 60, 256, seed=23).to(DEV)
    outs = {}
    for token_kernel in (False, True):
        for use_graph in (False, True):
            dec = Decoder(m, batch=B, use_graph=use_graph, token_kernel=token_kernel)
            assert dec._fused_ok() and dec._token_ok() == token_kernel
            assert dec.launches_per_token == (2 if token_kernel else 3 + 5 * m.layers)
            lg = [dec.prefill(ids[:, :40])]
            for t in range(40, 60):                                   # crosses the window edge (ctx 32): the position wraps
                lg.append(dec.step(ids[:, t]).clone())
            outs[(token_kernel, use_graph)] = (torch.stack(lg, 1), [st[0].clone() for st in dec.states])
    ref_lg, ref_S = outs[(False, False)]
    for key, (lg, S) in outs.items():
        close(lg, ref_lg, 2e-2, f"logits one-launch={key[0]} graph={key[1]}")
        for a, b in zip(S, ref_S):
            close(a, b, 5e-3, f"state one-launch={key[0]} graph={key[1]}")
    # the one-launch step repeats the chained kernels' arithmetic: most logits agree to the bit
    same = (outs[(True, True)][0] == ref_lg).float().mean().item()
    assert same > 0.9, same
    assert healthy() == 0


def test_generate_through_the_one_launch_step():
    m, _, _ = small_lm("aspin", "ln", torch.bfloat16)
    prompt = synth.token_ids(2, 40, 256, seed=3).to(DEV)
    for temp in (0.0, 1.0):
        a = Decoder(m, batch=2).generate(prompt, 24, temp=temp, seed=5)
        b = Decoder(m, batch=2, token_kernel=False).generate(prompt, 24, temp=temp, seed=5)
        c = Decoder(m, batch=2, use_graph=False).generate(prompt, 24, temp=temp, seed=5)
        assert tuple(a.shape) == (2, 24)
        assert torch.equal(a, c)                                      # graph replay and eager launches draw the same ids
        assert (a == b).float().mean().item() > 0.9                   # and the chained kernels' ids
    d = Decoder(m, batch=2)
    first = d.generate(prompt, 8, temp=0.0)
    again = d.generate(prompt, 8, temp=0.0)                           # the decoder, its table and its counters are reusable
    assert torch.equal(first, again)
    assert healthy() == 0


def test_changed_weights_retire_the_table():
    m, _, _ = small_lm("aspin", "rms", torch.bfloat16)
    prompt = synth.token_ids(1, 40, 256, seed=4).to(DEV)
    d = Decoder(m, batch=1)
    d.prefill(prompt); lg0 = d.step(prompt[:, -1]).clone()
    with torch.no_grad():
        m.mix[0].o.weight.mul_(0.5)                                   # the folded output weight is rebuilt, at a new address
    d.prefill(prompt); lg1 = d.step(prompt[:, -1]).clone()
    ref = Decoder(m, batch=1, token_kernel=False); ref.prefill(prompt)
    close(lg1, ref.step(prompt[:, -1]), 2e-2, "after the update")
    assert not torch.equal(lg0, lg1)


def test_a_barrier_wait_that_runs_out_raises_the_flag_and_returns():
    """The grid barrier's failure path without a fault: one CTA waits, with a short limit, for arrivals that never come."""
    import ctypes
    assert healthy() == 0
    sync = torch.zeros(2, dtype=torch.int64, device=DEV)
    rc = _lib.lib().pgb_decode_token_wait_selftest(ctypes.c_void_p(sync.data_ptr()), 2000, None)
    assert rc == 0
    torch.cuda.synchronize()
    assert sync[0].item() == 1                                        # it did arrive
    assert healthy() == 81 and healthy() == 0                         # reported once, then clear
    x = torch.ones(8, device=DEV)                                     # the context is still usable
    assert (x + 1).sum().item() == 16
