"""GPU parity tests of KV-cached greedy decode (Network.generate_greedy) against the reference's generation loop.

The reference recomputes the whole window for every token (demo.ipynb:1526-1533).  Greedy sequences fork at the
first near-tie, so sequences are compared (a) step by step against the literal reference loop until the first
position the tie rule excuses, and (b) teacher-forced: the emitted sequence is fed once through the oracle, and
every emitted token must be the oracle's arg-max at the previous position unless the oracle's top-2 gap is below the
tolerance (valid because the model is causal)."""
import numpy as np
import pytest

from conftest import TOL
from oracle import forward_np as onp
from torchless_nn_b200 import workloads as wl

pytestmark = pytest.mark.gpu


def _teacher_forced(spec, params, seq, tol_rel):
    """Oracle logits of the emitted sequences fed once (causal model): arg-max, top, runner-up per position and the
    absolute tolerance."""
    logits = onp.gpt_forward(spec, params, seq[:, :-1])
    a, top, second = onp.top2(logits)
    return a, top, second, tol_rel * float(np.abs(logits).max())


def _teacher_forced_ok(spec, params, seq, n_prompt, tol_rel, also=None):
    """seq: (B, T) emitted tokens (prompt + continuation).  Every emitted token must be the oracle's arg-max at the
    previous position unless the oracle's top-2 gap is below the tolerance.  `also` (B, T-1): tokens of another path
    of the engine for the same inputs (the prefill arg-max), held to the same rule at every position."""
    a, top, second, tol = _teacher_forced(spec, params, seq, tol_rel)
    emitted = seq[:, n_prompt:]
    ref = a[:, n_prompt - 1:]
    differ = emitted != ref
    excused = (top - second)[:, n_prompt - 1:] < tol
    if also is not None:
        ok, n_diff, n_bad = onp.tokens_match(also, a, top, second, tol)
        assert ok, f"prefill arg-max: {n_bad} of {n_diff} differing tokens are not excused by the tie rule"
    return int((differ & ~excused).sum()), int(differ.sum())


def _first_fork_is_excused(spec, params, one, other, tol_rel):
    """Two greedy continuations of the same prompt must agree up to the first position where the oracle, fed their
    common prefix, has a top-2 gap below the tolerance; after a near-tie they may go different ways."""
    same = one == other
    if same.all():
        return
    t = int(np.argmin(same))
    lg = onp.gpt_forward(spec, params, one[None, :t].astype(np.int64))[0, -1]
    srt = np.sort(lg)
    assert srt[-1] - srt[-2] < tol_rel * np.abs(lg).max(), f"sequences fork at position {t} on a clear arg-max"


def test_decode_c1_shape_tf32(engine):
    from torchless_nn_b200.models import build_seeded
    spec, net = build_seeded("c1")
    try:
        params = wl.seeded_params(spec)
        prompts = wl.make_inputs(spec, 6)[:, :20]
        out = net.generate_greedy(prompts, 40).get()
        assert out.shape == (6, 60) and out.dtype == np.int32
        assert np.array_equal(out[:, :20], prompts)
        bad, n = _teacher_forced_ok(spec, params, out.astype(np.int64), 20, TOL["tf32"])
        assert bad == 0, f"{bad} of {n} differing tokens are not excused by the tie rule"
        # literal reference loop on two prompts, compared until the first excused fork
        ref = onp.greedy_decode(spec, params, prompts[:2].astype(np.int64), 12)
        for b in range(2):
            same = out[b, :32] == ref[b]
            if not same.all():
                t = int(np.argmin(same))
                lg = onp.gpt_forward(spec, params, ref[b:b + 1, :t])[0, -1]
                srt = np.sort(lg)
                assert srt[-1] - srt[-2] < TOL["tf32"] * np.abs(lg).max()
        # decode and prefill agree with each other through the oracle: the arg-max of a full forward over the emitted
        # sequence obeys the same tie rule at every position
        tf = net.predict_tokens(out[:, :-1]).get()
        _teacher_forced_ok(spec, params, out.astype(np.int64), 20, TOL["tf32"], also=tf)
        # single new token, batch of one
        one = net.generate_greedy(prompts[:1], 1).get()
        assert one.shape == (1, 21) and one[0, 20] == out[0, 20]
        # beyond the context the window slides like the reference's loop (demo.ipynb:1528): 120 + 14 > 128
        long_prompts = wl.make_inputs(spec, 2)[:, :120]
        slid = net.generate_greedy(long_prompts, 14).get()
        assert slid.shape == (2, 134) and np.array_equal(slid[:, :120], long_prompts)
        ref_slid = onp.greedy_decode(spec, params, long_prompts.astype(np.int64), 14)
        for b in range(2):
            same = slid[b] == ref_slid[b]
            if not same.all():
                t = int(np.argmin(same))
                lg = onp.gpt_forward(spec, params, ref_slid[b:b + 1, max(0, t - spec.context):t])[0, -1]
                srt = np.sort(lg)
                assert srt[-1] - srt[-2] < TOL["tf32"] * np.abs(lg).max()
        with pytest.raises(ValueError):
            net.generate_greedy(prompts, 0)
        engine.set_precision("bf16")
        out_b = net.generate_greedy(prompts, 16).get()
        bad, n = _teacher_forced_ok(spec, params, out_b.astype(np.int64), 20, TOL["bf16"])
        assert bad == 0
    finally:
        engine.set_precision("tf32")


@pytest.fixture(scope="module")
def c4(engine):
    from torchless_nn_b200.models import build_seeded
    spec, net = build_seeded("c4")
    yield spec, net
    engine.set_precision("tf32")


def test_decode_c4_vs_reference_loop(engine, golden, c4):
    """Golden fixture: the reference's own recompute loop (arg-max) on 2 prompts x 24 steps."""
    spec, net = c4
    engine.set_precision("bf16")
    g = golden("c4")
    n_p, steps = int(g["n_prompts"]), int(g["steps"])
    prompts = wl.make_inputs(spec, n_p)
    out = net.generate_greedy(prompts, steps).get()
    tol = TOL["bf16"] * float(g["max_abs"])
    for b in range(n_p):
        for t in range(steps):
            if out[b, spec.seq_len + t] != g["tokens"][b, spec.seq_len + t]:
                assert g["top"][b, t] - g["second"][b, t] < tol, f"prompt {b} forks at step {t} on a clear arg-max"
                break


def test_decode_c4_full_size(engine, c4):
    """Full configuration: 64 prompts of 128 tokens, 256 new tokens each."""
    spec, net = c4
    engine.set_precision("bf16")
    prompts = wl.make_inputs(spec)
    out = net.generate_greedy(prompts, wl.C4_NEW_TOKENS).get()
    assert out.shape == (64, 384)
    assert np.array_equal(out[:, :128], prompts)
    assert out.min() >= 0 and out.max() < spec.vocab
    # batch rows are independent: a row decoded alone gives the same tokens
    params = wl.seeded_params(spec)
    alone = net.generate_greedy(prompts[7:8], 48).get()
    _first_fork_is_excused(spec, params, alone[0], out[7, :176], TOL["bf16"])
    # teacher-forced against the oracle on two sequences (causal: one forward per sequence), decode tokens and the
    # prefill path's arg-max of the same sequences
    tf = net.predict_tokens(out[:, :-1]).get()
    bad, n = _teacher_forced_ok(spec, params, out[:2].astype(np.int64), 128, TOL["bf16"], also=tf[:2])
    assert bad == 0, f"{bad} of {n} differing tokens are not excused by the tie rule"
    # decode against this engine's own prefill path on every fourth sequence: a decoded token may differ from the
    # prefill arg-max only where the prefill logits' own top-2 gap is inside the tolerance
    for r0 in range(0, 64, 16):
        rows = np.arange(r0, r0 + 16, 4)
        logits = net.predict_logits(out[rows, :-1]).get()
        a, top, second = onp.top2(logits)
        tol = TOL["bf16"] * float(np.abs(logits).max())
        differ = out[rows, 128:] != a[:, 127:]
        excused = (top - second)[:, 127:] < tol
        assert not (differ & ~excused).any(), f"{int((differ & ~excused).sum())} decode tokens differ from prefill on a clear arg-max"


def test_decode_with_a_long_cache(engine):
    """The single-query attention keeps nothing per cached position in shared memory (one pass, online softmax), so the
    cache length is bounded by the context only: caches of 16000 and 60000 positions give the tokens of a short one."""
    import ctypes as C
    from torchless_nn_b200 import backend
    from torchless_nn_b200._lib import lib, check
    from torchless_nn_b200.activations import GeLU
    from torchless_nn_b200.device_array import DeviceArray, as_token_ids
    from torchless_nn_b200.layers import TransformerBlock, LayerNorm
    from torchless_nn_b200.network import Network, GPTPlan
    from torchless_nn_b200.transformer_adapters import GPTEmbeddingTable, GPTEmbedFront, GPTEmbedBack, _ids_code
    for precision in ("tf32", "bf16"):
        engine.set_precision(precision)
        try:
            table = GPTEmbeddingTable(50, 64)
            net = Network([GPTEmbedFront(table, 70000), TransformerBlock(64, 70000, 2, GeLU, decoder=True),
                           LayerNorm(64), GPTEmbedBack(table)])
            net.set_eval(True)
            prompts = np.random.default_rng(5).integers(0, 50, (3, 9)).astype(np.int32)
            want = net.generate_greedy(prompts, 6).get()[:, 9:]              # cache of 15 positions
            m, keep, V = GPTPlan.match(net.layers).model()
            ids = as_token_ids(prompts)

            def run(max_len):
                first, rest, dec = DeviceArray((3,), np.int32), DeviceArray((3, 5), np.int32), C.c_void_p()
                check(lib.tlnn_decode_begin(backend.ctx(), C.byref(m), ids.ptr, _ids_code(ids), 3, 9, max_len, first.ptr, C.byref(dec)))
                try:
                    check(lib.tlnn_decode_run(dec, first.ptr, 5, rest.ptr))
                    return np.concatenate([first.get()[:, None], rest.get()], axis=1)
                finally:
                    lib.tlnn_decode_end(dec)

            assert np.array_equal(run(16000), want)
            assert np.array_equal(run(60000), want)
        finally:
            engine.set_precision("tf32")
