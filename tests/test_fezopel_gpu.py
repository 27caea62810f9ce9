"""The Fezopel decoder on the GPU against the plain float64 implementation in `plain_fezopel`: each mechanism alone
through its kernels, then whole models of several small shapes through the runner (prompts whole, tails token by token,
portions down to two tokens, mixed batches with pages and slots used again), and greedy generation through `Engine`.
The test models are random; where random weights would hide a fault the inputs are made so that it shows."""
import math

import numpy as np
import pytest
import torch

import helpers
import plain_fezopel as pf
import plain_model as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


# ---- small shapes -----------------------------------------------------------------------------------------------------
def att(heads, kv, dim, vdim, window, rot, base, scale):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": window},
                                           "rot": {"base": base, "dims": rot}, "scale": scale}}


def gla(heads, dim, vdim, tau, rank):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}}


def delta(heads, kv, dim, vdim, conv, rank, gate_rank):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv,
                                               "rank": rank, "gate_rank": gate_rank}}


def with_ff(layer, ff):
    return dict(layer, mlp={"kind": "dense", "ff": ff} if ff else None)


SHAPES = {
    # a recurrence first, two attention layers that differ in everything (two page groups), values narrower and wider than keys
    "P": {"architecture": "Fezopel", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "layers": [
        with_ff(gla(2, 24, 16, 8.0, 8), 0),
        with_ff(att(4, 1, 32, 16, 20, 16, 10000.0, 0.2), 96),
        with_ff(delta(4, 2, 16, 24, 3, 8, 4), 80),
        with_ff(att(2, 2, 16, 16, 37, 16, 500000.0, 0.25), 0)]},
    # sizes that are 1 or equal to one another: one head everywhere, two taps, a window of five, tau 1
    "Q": {"architecture": "Fezopel", "vocab": 61, "width": 40, "norm": {"eps": 1e-6}, "layers": [
        with_ff(delta(1, 1, 8, 8, 2, 8, 8), 40),
        with_ff(att(1, 1, 8, 24, 5, 4, 100.0, 1.0), 0),
        with_ff(gla(1, 8, 8, 1.0, 8), 40)]},
    # head size 64 and wider rows: prompts of a few hundred tokens send the products through the tcgen05 kernels
    "R": {"architecture": "Fezopel", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "layers": [
        with_ff(att(6, 3, 64, 64, 150, 32, 500000.0, 0.11), 256),
        with_ff(gla(4, 32, 64, 16.0, 16), 0),
        with_ff(delta(2, 1, 64, 32, 4, 16, 16), 0)]},
    # nothing is a multiple of 4: every kernel's path for odd widths, products on the plain kernel in both dtypes
    "S": {"architecture": "Fezopel", "vocab": 77, "width": 50, "norm": {"eps": 1e-6}, "layers": [
        with_ff(att(3, 3, 10, 6, 7, 6, 50.0, 0.3), 30),
        with_ff(gla(2, 20, 9, 3.0, 5), 0),
        with_ff(delta(3, 1, 12, 10, 5, 7, 3), 22)]},
    # no attention at all (no pages, only state slots), and nothing but attention (two layers of one page group, no slots)
    "T": {"architecture": "Fezopel", "vocab": 83, "width": 48, "norm": {"eps": 1e-5}, "layers": [
        with_ff(delta(2, 2, 16, 16, 4, 8, 8), 64),
        with_ff(gla(3, 16, 8, 4.0, 8), 0)]},
    "U": {"architecture": "Fezopel", "vocab": 83, "width": 48, "norm": {"eps": 1e-5}, "layers": [
        with_ff(att(3, 1, 16, 16, 9, 8, 10000.0, 0.25), 0),
        with_ff(att(3, 1, 16, 16, 9, 8, 10000.0, 0.25), 64)]},
}
SEEDS = {"P": 11, "Q": 12, "R": 13, "S": 14, "T": 15, "U": 16}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from boring_llm_b200 import FezopelConfig, write_random_model
    made = {}

    def get(name, std=0.25):
        key = (name, std)
        if key not in made:
            d = str(tmp_path_factory.mktemp(f"fez_{name}"))
            write_random_model(d, FezopelConfig.from_dict(SHAPES[name]), SEEDS[name], "bfloat16", std)
            made[key] = d
        return made[key]
    return get


def plain_logits(folder, tokens):
    cfg, W = plain.read_model_folder(folder)
    return pf.forward(cfg, W, tokens).numpy()


def check_trace(folder, dtype, reqs, steps, max_tokens, what, tol=None, **kw):
    outputs, runner = helpers.run_inprocess(folder, dtype, steps, max_tokens, **kw)
    rows = helpers.collect_rows(steps, outputs)
    for rid, toks in reqs.items():
        want = plain_logits(folder, toks)
        got = np.stack([rows[(rid, p)] for p in range(len(toks))])
        helpers.assert_close(got, want, dtype, f"{what} {rid}", tol=tol, mean_tol=None if tol is None else tol / 4)
    return runner


def solo_steps(reqs, cut):
    steps, n0 = [], 0
    for i, (rid, toks) in enumerate(reqs.items()):
        s = helpers.solo_trace(rid, toks, cut(toks, i), n0)
        steps += s
        n0 += len(s)
    return steps


# bfloat16 against pure float64: activations are rounded to 8 bits between kernels, and the test weights are sharp
BF16_TOL = 6e-2


# ---- whole models ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["P", "Q", "S"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_whole_tails_singly_and_portions(folders, name, dtype):
    folder = folders(name, 0.25 if dtype == "float32" else 0.1)
    vocab = SHAPES[name]["vocab"]
    reqs = {f"r{i}": helpers.random_tokens(vocab, n, 100 + i) for i, n in enumerate([1, 2, 19, 75, 130])}
    tol = None if dtype == "float32" else BF16_TOL
    check_trace(folder, dtype, reqs, solo_steps(reqs, lambda t, i: helpers.cut_whole(t)), 256, f"{name} whole", tol)
    check_trace(folder, dtype, reqs, solo_steps(reqs, lambda t, i: helpers.cut_tail_singly(t, 45)), 256, f"{name} tail", tol)
    check_trace(folder, dtype, reqs, solo_steps(reqs, lambda t, i: helpers.cut_varying(t, i)), 256, f"{name} portions", tol)
    check_trace(folder, dtype, reqs, solo_steps(reqs, lambda t, i: [2] * (len(t) // 2) + [1] * (len(t) % 2)), 256,
                f"{name} pairs", tol)


@pytest.mark.parametrize("name", ["P", "Q", "S", "T", "U"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_reuse_pages_and_slots(folders, name, dtype):
    folder = folders(name, 0.25 if dtype == "float32" else 0.1)
    vocab = SHAPES[name]["vocab"]
    reqs = {f"m{i}": helpers.random_tokens(vocab, n, 200 + i) for i, n in enumerate([33, 7, 90, 41, 2, 64, 17, 58])}
    steps, peak = helpers.mixed_trace(reqs, seed=5, max_live=3)
    runner = check_trace(folder, dtype, reqs, steps, peak, f"{name} mixed", None if dtype == "float32" else BF16_TOL,
                         debug_poison=True)
    # eight requests went through at most three live at a time: slots and pages were handed out again
    assert all(hw <= runner.cache.num_pages for hw in runner.cache.stats()["pages_high_water"])
    assert (len(runner.cache.state_groups) >= 1) == (name != "U") and (len(runner.cache.paged_groups) >= 1) == (name != "T")


def test_float32_does_not_depend_on_the_cut_or_the_batch(folders):
    """The same position's logits from a whole prompt, from portions and from a mixed batch agree to rounding."""
    folder = folders("P")
    reqs = {f"c{i}": helpers.random_tokens(97, n, 300 + i) for i, n in enumerate([50, 21, 77])}
    a, _ = helpers.run_inprocess(folder, "float32", solo_steps(reqs, lambda t, i: helpers.cut_whole(t)), 256)
    whole = helpers.collect_rows(solo_steps(reqs, lambda t, i: helpers.cut_whole(t)), a)
    steps, peak = helpers.mixed_trace(reqs, seed=9, max_live=3)
    b, _ = helpers.run_inprocess(folder, "float32", steps, peak)
    mixed = helpers.collect_rows(steps, b)
    for key, row in whole.items():
        assert np.abs(row - mixed[key]).max() <= 2e-5 * max(1.0, np.abs(row).max()), key


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_every_window(folders, dtype):
    folder = folders("P", 0.25 if dtype == "float32" else 0.1)
    toks = helpers.random_tokens(97, 330, 7)
    reqs = {"long": toks}
    steps = helpers.solo_trace("long", toks, [30] + [1] * 300)
    check_trace(folder, dtype, reqs, steps, 384, "long decoding", None if dtype == "float32" else BF16_TOL)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wide_shape_on_the_tensor_core_products(folders, dtype):
    """Prompts of 300 and 90 tokens: in bfloat16 the joined projections run on tcgen05 (pairs of SMs from 256 rows, one
    SM from 65), decode steps replay captured graphs; a window wider than a page and than a key block."""
    folder = folders("R", 0.25 if dtype == "float32" else 0.06)
    reqs = {"w0": helpers.random_tokens(300, 300, 1), "w1": helpers.random_tokens(300, 90, 2)}
    tol = None if dtype == "float32" else BF16_TOL
    steps = solo_steps(reqs, lambda t, i: helpers.cut_tail_singly(t, 24))
    runner = check_trace(folder, dtype, reqs, steps, 512, "wide tail", tol)
    runner.check_kernels()
    steps, peak = helpers.mixed_trace(reqs, seed=3, max_live=2)
    check_trace(folder, dtype, reqs, steps, peak, "wide mixed", tol).check_kernels()


def test_captured_steps_replay_the_same_bits(folders):
    """bfloat16: the second pass over a trace replays captured graphs (decode steps and padded general steps) and must
    give what the first pass, launched kernel by kernel, gave, state slots and pages having been used in between."""
    folder = folders("P", 0.1)
    reqs = {f"g{i}": helpers.random_tokens(97, n, 400 + i) for i, n in enumerate([40, 23, 31])}
    steps, peak = helpers.mixed_trace(reqs, seed=4, max_live=3)
    twice = steps + [dict(s, step=s["step"] + len(steps)) for s in steps]
    out, runner = helpers.run_inprocess(folder, "bfloat16", twice, peak, step_graph_after=1)
    assert runner.graph_steps > 0
    for s in steps:
        if s["step"] in out:
            np.testing.assert_array_equal(out[s["step"]], out[s["step"] + len(steps)])


def test_greedy_generation_through_the_engine(folders):
    import boring_llm_b200 as b
    for name, dtype, std in (("P", "float32", 0.25), ("Q", "bfloat16", 0.1)):
        folder = folders(name, std)
        vocab = SHAPES[name]["vocab"]
        prompts = [helpers.random_tokens(vocab, n, 500 + n) for n in (5, 26, 61)]
        eng = b.Engine(folder, dtype=dtype, ctx_size=128, max_num_seqs=2, max_tokens=192, prefill_chunk=16)
        outs = eng.generate(prompts, n_predict=12, ignore_eos=True)
        for p, o in zip(prompts, outs):
            assert len(o) == 12
            logits = plain_logits(folder, p + o)
            for i, tok in enumerate(o):
                row = logits[len(p) - 1 + i]
                gap = row.max() - row[tok]
                assert gap <= (1e-4 if dtype == "float32" else 0.05) * np.abs(logits).max(), (name, i, gap)


# ---- mechanisms alone --------------------------------------------------------------------------------------------------
def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g, dtype=torch.float64) * scale)


def test_layer_norm_gated_residual_depth_mix_and_activations():
    from boring_llm_b200.kernels import ops
    for rows, d in ((5, 40), (33, 129), (2, 1)):
        x, w, b = rnd(rows, d, seed=1, scale=3.0) + 2.0, rnd(d, seed=2) + 1.0, rnd(d, seed=3)
        xg, wg, bg = x.float().to(DEV), w.float().to(DEV), b.float().to(DEV)
        out = torch.empty(rows, d, device=DEV)
        ops.layernorm(xg, wg, bg, 1e-5, out)
        np.testing.assert_allclose(out.cpu().numpy(), pf.layer_norm(x, w, b, 1e-5).numpy(), atol=2e-5, rtol=1e-5)
        idx = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
        out2 = torch.empty(2, d, device=DEV)
        ops.layernorm(xg, wg, None, 1e-5, out2, idx)
        np.testing.assert_allclose(out2.cpu().numpy(), pf.layer_norm(x[[rows - 1, 0]], w, 0.0, 1e-5).numpy(), atol=2e-5, rtol=1e-5)
        sub, gate = rnd(rows, d, seed=4, scale=2.0), rnd(rows, d + 3, seed=5, scale=2.0)
        stream = xg.clone()
        ops.gated_norm_residual(stream, sub.float().to(DEV), gate.float().to(DEV)[:, 1:d + 1], wg, bg, 1e-5)
        want = x + pf.layer_norm(sub * torch.sigmoid(gate[:, 1:d + 1]), w, b, 1e-5)
        np.testing.assert_allclose(stream.cpu().numpy(), want.numpy(), atol=3e-5, rtol=1e-5)
        gb = rnd(d, seed=9)                              # the gate's bias added by the kernel, the logits without it
        stream = xg.clone()
        ops.gated_norm_residual(stream, sub.float().to(DEV), (gate[:, 1:d + 1] - gb).float().to(DEV).contiguous(), wg, None, 1e-5,
                                gb.float().to(DEV))
        want = x + pf.layer_norm(sub * torch.sigmoid(gate[:, 1:d + 1]), w, 0.0, 1e-5)
        np.testing.assert_allclose(stream.cpu().numpy(), want.numpy(), atol=3e-5, rtol=1e-5)
    streams, c = rnd(5, 7, 12, seed=6), rnd(4, seed=7)
    sg = streams.float().to(DEV)
    ops.depth_mix(sg, c.float().to(DEV), 4, sg[4])
    np.testing.assert_allclose(sg[4].cpu().numpy(), torch.einsum("j,jtd->td", c, streams[:4]).numpy(), atol=1e-5)
    z = rnd(9, 31, seed=8, scale=3.0)
    for act, fn in ((ops.ACT_GELU_ERF, pf.gelu_erf), (ops.ACT_SILU, pf.silu),
                    (ops.ACT_GELU_TANH, lambda v: 0.5 * v * (1 + torch.tanh(math.sqrt(2 / math.pi) * (v + 0.044715 * v ** 3))))):
        out = torch.empty(9, 31, device=DEV)
        ops.activation(z.float().to(DEV), out, act)
        np.testing.assert_allclose(out.cpu().numpy(), fn(z).numpy(), atol=2e-6, rtol=1e-5)


def paged(x, page, n_pages, order):
    """x [T, G, d] of one request -> (cache [n_pages + 1, G, page, d] filled with NaN elsewhere, block table row)."""
    T, G, d = x.shape
    cache = torch.full((n_pages + 1, G, page, d), float("nan"), dtype=torch.float32)
    table = []
    for i in range(-(-T // page)):
        p = order[i]
        table.append(p)
        n = min(page, T - i * page)
        cache[p, :, :n] = x[i * page:i * page + n].permute(1, 0, 2).float()
        cache[p, :, n:] = 0.0
    return cache, table


@pytest.mark.parametrize("H,G,dk,dv,window", [(4, 2, 16, 16, 0), (3, 1, 24, 8, 21), (2, 2, 8, 40, 16), (1, 1, 32, 32, 1)])
def test_sink_attention_kernel_with_planted_keys(H, G, dk, dv, window):
    """Keys at chosen distances get a score that dominates: just inside and just outside the window, at page borders,
    the first token, far back. Pages are scattered and the unused rest of the pool is NaN."""
    from boring_llm_b200.kernels import ops
    T, page = 150, 16
    q, k, v = rnd(T, H, dk, seed=1), rnd(T, G, dk, seed=2), rnd(T, G, dv, seed=3)
    sinks = rnd(H, seed=4, scale=2.0)
    gate = rnd(T, H + 2, seed=5)
    for qi, kj in ((149, 0), (149, 149 - (window or 100) + 1), (149, 149 - (window or 100)), (100, 96), (100, 95), (64, 63),
                   (64, 48), (64, 47), (33, 32), (16, 15), (16, 0)):
        kj = max(0, kj)
        k[kj] = k[kj] * 0 + q[qi, 0] / q[qi, 0].norm() * 6.0          # q[qi] . k[kj] large for head 0's group
    want = pf.sink_window_attention(q, k, v, 0.3, window, sinks) * torch.sigmoid(gate[:, 1:H + 1])[:, :, None]
    order = list(np.random.default_rng(0).permutation(12))
    kc, table = paged(k, page, 12, order)
    vc, _ = paged(v, page, 12, order)
    # the request's tokens arrive as two portions and then singly: a step's queries see the keys of the steps before
    out = torch.empty(T, H * dv, device=DEV)
    cuts = [90, 50] + [1] * 10
    at = 0
    tb = torch.tensor([table + [-1] * (16 - len(table))], dtype=torch.int32, device=DEV)
    for n in cuts:
        sl = slice(at, at + n)
        o = torch.empty(n, H * dv, device=DEV)
        ops.attention_plain(q[sl].reshape(n, H * dk).float().to(DEV).contiguous(), kc.to(DEV), vc.to(DEV),
                            torch.zeros(n, dtype=torch.int32, device=DEV), torch.tensor([0, n], dtype=torch.int32, device=DEV),
                            torch.tensor([at + n], dtype=torch.int32, device=DEV), tb, o, H, window, 0.3,
                            sinks.float().to(DEV), gate.float().to(DEV)[sl, 1:H + 1])
        out[sl] = o
        at += n
    got = out.cpu().numpy().reshape(T, H, dv)
    assert np.isfinite(got).all()
    np.testing.assert_allclose(got, want.numpy(), atol=3e-5, rtol=2e-4)
    # losing the planted key would have shown: with it masked the output of that query moves by far more than the tolerance
    k2 = k.clone(); k2[0] = 0
    moved = (pf.sink_window_attention(q, k2, v, 0.3, window, sinks)[16] - pf.sink_window_attention(q, k, v, 0.3, window, sinks)[16]).abs().max()
    if window == 0 or window > 16:
        assert moved > 1e-2


def test_a_large_sink_takes_the_weight_and_none_leaves_plain_softmax():
    q, k, v = rnd(6, 2, 8, seed=1), rnd(6, 1, 8, seed=2), rnd(6, 1, 8, seed=3)
    none = pf.sink_window_attention(q, k, v, 0.5, 0, torch.full((2,), -1e9, dtype=torch.float64))
    s = torch.einsum("ihd,jd->hij", q, k[:, 0]) * 0.5
    s = s.masked_fill(torch.triu(torch.ones(6, 6, dtype=torch.bool), 1), float("-inf"))
    np.testing.assert_allclose(none.numpy(), torch.einsum("hij,jd->ihd", torch.softmax(s, -1), v[:, 0]).numpy(), atol=1e-12)
    big = pf.sink_window_attention(q, k, v, 0.5, 0, torch.full((2,), 40.0, dtype=torch.float64))
    assert big.abs().max() < 1e-10


@pytest.mark.parametrize("H,G,dk,dv,rot,layout", [(4, 2, 16, 8, 16, 1), (3, 1, 12, 20, 6, 1), (2, 2, 8, 8, 0, 1), (2, 1, 16, 16, 8, 0)])
def test_whole_projection_norm_rotation_and_cache_write(H, G, dk, dv, rot, layout):
    from boring_llm_b200.kernels import ops
    from boring_llm_b200.parts import RotaryTable
    T, page = 37, 16
    pos0 = 1000                                                    # angles of a long context
    n_in = H * dk + G * dk + G * dv + 5
    proj = rnd(T, n_in, seed=1, scale=2.0)
    qw, kw = rnd(H * dk, seed=2) + 1.0, rnd(G * dk, seed=3) + 1.0
    table = RotaryTable(dk, 10000.0, n_rot=rot, pairs="interleaved" if layout else "halves").to(DEV)
    positions = torch.arange(pos0, pos0 + T, dtype=torch.int32, device=DEV)
    n_pages = -(-(pos0 + T) // page)
    tb = torch.arange(n_pages, dtype=torch.int32, device=DEV)[None, :].contiguous()
    kc = torch.zeros(n_pages, G, page, dk, device=DEV)
    vc = torch.zeros(n_pages, G, page, dv, device=DEV)
    q_out = torch.empty(T, H * dk, device=DEV)
    ops.qk_norm_rope_write(proj.float().to(DEV), H * dk, H * dk + G * dk, qw.float().to(DEV), kw.float().to(DEV), 1e-6, positions,
                           torch.zeros(T, dtype=torch.int32, device=DEV), tb, table.inv_freq, rot // 2, layout, q_out, kc, vc,
                           H, G, dk, dv)
    q = pf.rms_unit(proj[:, :H * dk], 1e-6) * qw
    k = pf.rms_unit(proj[:, H * dk:H * dk + G * dk], 1e-6) * kw
    p = list(range(pos0, pos0 + T))
    if layout:
        qr = pf.rotate_interleaved(q.reshape(T, H, dk), p, 10000.0, rot) if rot else q.reshape(T, H, dk)
        kr = pf.rotate_interleaved(k.reshape(T, G, dk), p, 10000.0, rot) if rot else k.reshape(T, G, dk)
    else:
        f = plain.rope_inv_freq(rot, 10000.0)
        def halves(x):
            out = x.clone()
            ang = torch.tensor(p, dtype=torch.float64)[:, None] * torch.from_numpy(f.astype(np.float64))[None, :]
            c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            a, b = x[..., :rot // 2], x[..., rot // 2:rot]
            out[..., :rot // 2] = a * c - b * s
            out[..., rot // 2:rot] = b * c + a * s
            return out
        qr, kr = halves(q.reshape(T, H, dk)), halves(k.reshape(T, G, dk))
    np.testing.assert_allclose(q_out.cpu().numpy().reshape(T, H, dk), qr.numpy(), atol=2e-4, rtol=1e-4)
    rows = torch.tensor(p)
    got_k = kc.cpu()[rows // page, :, rows % page]                    # [T, G, dk]
    got_v = vc.cpu()[rows // page, :, rows % page]
    np.testing.assert_allclose(got_k.numpy(), kr.numpy(), atol=2e-4, rtol=1e-4)
    np.testing.assert_allclose(got_v.numpy(), proj[:, H * dk + G * dk:H * dk + G * dk + G * dv].reshape(T, G, dv).float().numpy(), atol=0)


@pytest.mark.parametrize("rule", ["gla", "delta"])
@pytest.mark.parametrize("H,G,dk,dv", [(2, 2, 24, 16), (3, 1, 20, 9), (1, 1, 64, 40), (2, 1, 130, 8)])
def test_recurrence_kernel_in_portions_with_slots_used_again(rule, H, G, dk, dv):
    """Two requests in one batch (unequal portions, one sitting a step out), their states in slots that an earlier request
    has left dirty and that were cleared on admission; the state decays slowly, so a token 200 steps back still counts."""
    from boring_llm_b200.kernels import ops
    if rule == "gla":
        G = H
    lens = {"a": 230, "b": 57}
    data = {}
    for i, (rid, T) in enumerate(lens.items()):
        q, k = rnd(T, G, dk, seed=10 + i, scale=0.5), rnd(T, G, dk, seed=20 + i, scale=0.5)
        if rule == "delta":
            k = k / k.norm(dim=-1, keepdim=True)
        v, z, beta = rnd(T, H, dv, seed=30 + i), rnd(T, H, dk, seed=40 + i) + 3.0, rnd(T, H, seed=50 + i)
        data[rid] = (q, k, v, z, beta)
    coef = torch.tensor([0.05 * (h + 1) for h in range(H)], dtype=torch.float64)
    want = {}
    rep = H // G
    for rid, (q, k, v, z, beta) in data.items():
        if rule == "gla":
            a = torch.exp(-coef[None, :, None] * pf.softplus(-z))
            want[rid] = pf.gated_linear_recurrence(q * 0.7, k, v, a)
        else:
            a = torch.exp(-coef[None, :, None] * pf.softplus(z))
            want[rid] = pf.delta_recurrence(q.repeat_interleave(rep, 1) * 0.7, k.repeat_interleave(rep, 1), v, a, torch.sigmoid(beta))
    n_state = H * dk * dv
    state = torch.full((4, n_state + 7), float("nan"), device=DEV)          # dirty slots, and room behind the matrix state
    slots = {"a": 2, "b": 0}
    for s in slots.values():
        state[s, :n_state].zero_()
    got = {rid: torch.zeros(T, H * dv) for rid, T in lens.items()}
    at = {"a": 0, "b": 0}
    plan = [{"a": 100, "b": 2}, {"a": 1}, {"b": 30, "a": 64}, {"a": 2, "b": 1}, {"b": 24, "a": 63}]
    for step in plan:
        rids = list(step)
        parts = [[t[at[r]:at[r] + step[r]] for t in data[r]] for r in rids]
        cat = lambda j, w: torch.cat([p[j].reshape(p[j].shape[0], w) for p in parts]).float().to(DEV).contiguous()
        q, k, v, z, beta = cat(0, G * dk), cat(1, G * dk), cat(2, H * dv), cat(3, H * dk), cat(4, H)
        T = q.shape[0]
        # the decays come out of the product that makes their pre-activation: here z = z . I + 0
        decay = torch.empty(T, H * dk, device=DEV)
        ops.gemm_plain_decay(z, torch.eye(H * dk, device=DEV), None, coef.float().to(DEV), dk, -1.0 if rule == "gla" else 1.0, decay)
        cu = torch.tensor(np.cumsum([0] + [step[r] for r in rids]), dtype=torch.int32, device=DEV)
        out = torch.empty(T, H * dv, device=DEV)
        ops.recurrent_scan(ops.RULE_GLA if rule == "gla" else ops.RULE_DELTA, q, k, v, decay, beta if rule == "delta" else None,
                           0.7, state, torch.tensor([slots[r] for r in rids], dtype=torch.int32, device=DEV), cu, out, H, G, dk, dv)
        o = out.cpu()
        t0 = 0
        for r in rids:
            got[r][at[r]:at[r] + step[r]] = o[t0:t0 + step[r]]
            t0 += step[r]; at[r] += step[r]
    assert at == lens
    for rid in lens:
        w = want[rid].reshape(lens[rid], H * dv).numpy()
        np.testing.assert_allclose(got[rid].numpy(), w, atol=2e-4 * max(1.0, np.abs(w).max()), rtol=2e-4)
    assert torch.isnan(state[1]).all() and torch.isnan(state[3]).all()          # nobody else's slot was touched
    assert torch.isnan(state[0, n_state:]).all()                                # nor the room behind a matrix state
    # the first token still counts at the end of request a: without it the last output differs
    q, k, v, z, beta = data["a"]
    if rule == "gla":
        a = torch.exp(-coef[None, :, None] * pf.softplus(-z))
        v2 = v.clone(); v2[0] = 0
        assert (pf.gated_linear_recurrence(q * 0.7, k, v2, a)[-1] - want["a"][-1]).abs().max() > 1e-3 * want["a"][-1].abs().max()


@pytest.mark.parametrize("taps,G,H,dk,dv", [(4, 2, 4, 8, 12), (2, 1, 1, 16, 16), (3, 1, 3, 6, 5), (1, 1, 2, 8, 8)])
def test_short_convolution_with_its_tail_in_the_slot(taps, G, H, dk, dv):
    from boring_llm_b200.kernels import ops
    C = 2 * G * dk + H * dv
    T = 23
    x = rnd(T, C + 6, seed=1)                          # the convolved channels are the first C of wider rows
    w = rnd(C, taps, seed=2)
    y = pf.silu(pf.short_conv(x[:, :C], w))
    qk = y[:, :2 * G * dk].reshape(T, 2 * G, dk)
    qk = qk / torch.sqrt((qk * qk).sum(-1, keepdim=True) + 1e-6)
    qk[:, :G] *= 0.25
    want = torch.cat([qk.reshape(T, -1), y[:, 2 * G * dk:]], 1)
    off = 11                                           # the tail lies behind other state in the slot
    state = torch.full((3, off + (taps - 1) * C), float("nan"), device=DEV)
    state[1].zero_()
    tail = state[:, off:]
    got = []
    at = 0
    for n in (1, 1, 2, 1, 3, 5, 2, 8):                # portions shorter than the taps among them
        xs = x[at:at + n].float().to(DEV).contiguous()
        out = torch.empty(n, C, device=DEV)
        slots = torch.tensor([1], dtype=torch.int32, device=DEV)
        cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
        ops.conv_silu_unit(xs, w.float().to(DEV), tail, slots, torch.zeros(n, dtype=torch.int32, device=DEV), cu, out,
                           2 * G, G, dk, 0.25, 1e-6)
        ops.conv_tail_update(xs, taps, tail, slots, cu, C)
        got.append(out.cpu())
        at += n
    assert at == T
    np.testing.assert_allclose(torch.cat(got).numpy(), want.numpy(), atol=3e-5, rtol=1e-4)
    assert torch.isnan(state[0]).all() and torch.isnan(state[1, :off].cpu()).sum() == 0


def test_head_norm_and_gates():
    from boring_llm_b200.kernels import ops
    T, H, dv = 7, 3, 20
    o, w, g = rnd(T, H * dv, seed=1, scale=4.0), rnd(dv, seed=2) + 1.0, rnd(T, H * dv + 4, seed=3)
    for kind, fn in ((ops.GATE_SILU, pf.silu), (ops.GATE_SIGMOID, torch.sigmoid)):
        out = torch.empty(T, H * dv, device=DEV)
        ops.head_norm_gate(o.float().to(DEV), w.float().to(DEV), g.float().to(DEV)[:, 2:2 + H * dv], kind, 1e-5, out, H, dv)
        want = (pf.rms_unit(o.reshape(T, H, dv), 1e-5) * w).reshape(T, H * dv) * fn(g[:, 2:2 + H * dv])
        np.testing.assert_allclose(out.cpu().numpy(), want.numpy(), atol=3e-5, rtol=1e-4)


@pytest.mark.parametrize("dh,H,G,window", [(64, 4, 2, 0), (64, 8, 1, 150), (32, 2, 2, 40), (128, 2, 1, 0)])
def test_sinks_and_gates_in_the_tensor_core_attention_kernels(dh, H, G, window):
    """Every bfloat16 attention kernel (prefill on mma.sync and on tcgen05, decode on mma.sync with one slice, with a
    cluster's slices and with slices merged through scratch, decode fed by TMA) with sinks so large that they take about
    half of every row's weight, and gates: a sink that was left out, or counted once per slice, doubles or halves rows."""
    from boring_llm_b200.kernels import ops
    from boring_llm_b200.parts.attention import attention_plan
    T, page = 300, 16
    bf = lambda x: x.to(torch.bfloat16).to(torch.float64)
    q, k, v = bf(rnd(T, H, dh, seed=1)), bf(rnd(T, G, dh, seed=2)), bf(rnd(T, G, dh, seed=3))
    scale = dh ** -0.5
    gate = rnd(T, H + 1, seed=5)
    # a sink near the log of the sum of the row's exponentials: about half the weight
    sinks = bf(torch.full((H,), math.log(min(T, window or T) / 2) + 0.5, dtype=torch.float64) + rnd(H, seed=4) * 0.3)
    want = (pf.sink_window_attention(q, k, v, scale, window, sinks) * torch.sigmoid(gate[:, :H])[:, :, None]).reshape(T, H * dh)
    no_sink = pf.sink_window_attention(q, k, v, scale, window, torch.full((H,), -1e9, dtype=torch.float64))
    assert (no_sink.reshape(T, -1)[-1].abs().max() > 1.3 * pf.sink_window_attention(q, k, v, scale, window, sinks).reshape(T, -1)[-1].abs().max())
    n_pages = 24
    order = list(np.random.default_rng(1).permutation(n_pages))
    kc, table = paged(k, page, n_pages, order)
    vc, _ = paged(v, page, n_pages, order)
    kc, vc = torch.nan_to_num(kc, nan=0.0).to(torch.bfloat16).to(DEV), torch.nan_to_num(vc, nan=0.0).to(torch.bfloat16).to(DEV)
    qg = q.reshape(T, H * dh).to(torch.bfloat16).to(DEV).contiguous()
    sg, gg = sinks.float().to(DEV), gate.float().to(DEV)[:, :H]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    tol = dict(atol=2e-2 * float(want.abs().max()), rtol=2e-2)
    # prefill: one request of T tokens
    plan = attention_plan([T], [T])
    tb = i32([table + [-1] * (32 - len(table))])
    out = torch.zeros(T, H * dh, dtype=torch.bfloat16, device=DEV)
    ops.attention_prefill(qg, kc, vc, i32([0, T]), i32([T]), tb, i32(plan.arrays["tiles64"]), out, H, window, scale, sg, gg)
    np.testing.assert_allclose(out.float().cpu().numpy(), want.numpy(), **tol)
    if ops.attention_prefill_tc_supported(torch.bfloat16, dh, page):
        out = torch.zeros(T, H * dh, dtype=torch.bfloat16, device=DEV)
        ops.attention_prefill_tc(qg, kc, vc, i32([0, T]), i32([T]), tb, i32(plan.arrays["tiles128"]), out, H, window, scale, sg, gg)
        ops.check_status()
        np.testing.assert_allclose(out.float().cpu().numpy(), want.numpy(), **tol)
    # decode: three requests on the same pages with contexts of 300, 170 and 33 tokens
    ctxs = [300, 170, 33]
    rows = [c - 1 for c in ctxs]
    qd = qg[rows].contiguous()
    gd = gate.float().to(DEV)[rows][:, :H]
    tb3 = tb.repeat(3, 1).contiguous()
    cu, cl, reqs = i32([0, 1, 2, 3]), i32(ctxs), i32([0, 1, 2])
    for splits, scratch in ((1, False), (4, False), (5, True)):
        out = torch.zeros(3, H * dh, dtype=torch.bfloat16, device=DEV)
        sc = torch.empty(ops.attention_decode_scratch(3, H, dh, splits), device=DEV) if scratch else None
        ops.attention_decode(qd, kc, vc, cu, cl, tb3, reqs, splits, out, H, window, scale, sc, sinks=sg, gate=gd)
        np.testing.assert_allclose(out.float().cpu().numpy(), want[rows].numpy(), err_msg=f"mma decode, {splits} slices", **tol)
    if ops.attention_decode_tma_supported(torch.bfloat16, dh, page):
        for splits in (1, 3):
            out = torch.zeros(3, H * dh, dtype=torch.bfloat16, device=DEV)
            ops.attention_decode_tma(qd, kc, vc, cu, cl, tb3, reqs, splits, out, H, window, scale, sg, gd)
            ops.check_status()
            np.testing.assert_allclose(out.float().cpu().numpy(), want[rows].numpy(), err_msg=f"TMA decode, {splits} slices", **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_row_chain_gives_the_bits_of_its_three_kernels(dtype):
    """Gate + norm + residual, the average over the streams and the next norm in one launch against the three launches."""
    from boring_llm_b200.kernels import ops
    T, d, n = 9, 136, 4
    streams = rnd(n + 1, T, d, seed=1).float().to(DEV)
    sub, gate = rnd(T, d, seed=2, scale=2.0).float().to(DEV), rnd(T, d + 8, seed=3).float().to(DEV)[:, 8:]
    gb, w, b = rnd(d, seed=4).float().to(DEV), (rnd(d, seed=5) + 1).float().to(DEV), rnd(d, seed=6).float().to(DEV)
    w2, b2, c = (rnd(d, seed=7) + 1).float().to(DEV), rnd(d, seed=8).float().to(DEV), rnd(n, seed=9).float().to(DEV)
    a = streams.clone()
    ops.gated_norm_residual(a[n - 1], sub, gate, w, b, 1e-5, gb)
    ops.depth_mix(a, c, n, a[n])
    ya = torch.empty(T, d, dtype=dtype, device=DEV)
    ops.layernorm(a[n], w2, b2, 1e-6, ya)
    f = streams.clone()
    yf = torch.empty(T, d, dtype=dtype, device=DEV)
    assert ops.norm_chain_supported(f[n - 1], gate)
    ops.norm_chain(f[n - 1], sub, gate, gb, (w, b, 1e-5), streams=f, coeffs=c, n=n, mix_out=f[n], then=(w2, b2, 1e-6), y=yf)
    assert torch.equal(a, f) and torch.equal(ya, yf)
    # the steps alone: only the residual; the residual and a norm of the same block
    g = streams.clone()
    ops.norm_chain(g[n - 1], sub, gate, gb, (w, b, 1e-5))
    assert torch.equal(g[n - 1], a[n - 1])
    yg = torch.empty(T, d, dtype=dtype, device=DEV)
    ops.norm_chain(g[0], sub, None, None, (w, None, 1e-5), then=(w2, None, 1e-6), y=yg)
    h = streams.clone()
    ops.gated_norm_residual(h[0], sub, None, w, None, 1e-5)
    yh = torch.empty(T, d, dtype=dtype, device=DEV)
    ops.layernorm(h[0], w2, None, 1e-6, yh)
    assert torch.equal(g[0], h[0]) and torch.equal(yg, yh)


@pytest.mark.parametrize("H,dk,dv", [(2, 16, 24), (1, 64, 40), (3, 48, 8)])
def test_long_portions_of_linear_attention_cut_into_parts(H, dk, dv):
    """Three requests in one step, of 700, 256 and 40 tokens (the last is too short to be cut), each from a state that an
    earlier step left: the parts run side by side and give what the walk in one piece gives, and the slots hold the same
    states afterwards."""
    from boring_llm_b200.kernels import ops
    lens = [700, 256, 40]
    T = sum(lens)
    q, k, v = rnd(T, H * dk, seed=1, scale=0.5), rnd(T, H * dk, seed=2, scale=0.5), rnd(T, H * dv, seed=3)
    a = torch.rand(T, H * dk, generator=torch.Generator().manual_seed(4), dtype=torch.float64) * 0.08 + 0.92
    start = rnd(3, H * dk * dv, seed=5)
    cu = torch.tensor(np.cumsum([0] + lens), dtype=torch.int32, device=DEV)
    slots = torch.tensor([2, 0, 1], dtype=torch.int32, device=DEV)
    assert ops.recurrent_scan_parts(ops.RULE_GLA, H, dk, dv, 2) > 1 and ops.recurrent_scan_parts(ops.RULE_DELTA, H, dk, dv, 2) > 1
    assert ops.recurrent_scan_parts(ops.RULE_DELTA, 2, 256, 64, 1) == 1           # the matrix fold takes key sizes up to 128
    assert ops.recurrent_scan_parts(ops.RULE_GLA, 64, 128, 512, 4) == 1          # enough blocks as it is: a cut would not pay
    results = []
    for parts in (1, ops.SCAN_MAX_PARTS, 5):
        state = torch.zeros(4, H * dk * dv, device=DEV)
        state[slots.long()] = start.float().to(DEV)
        out = torch.empty(T, H * dv, device=DEV)
        ops.recurrent_scan(ops.RULE_GLA, q.float().to(DEV), k.float().to(DEV), v.float().to(DEV), a.float().to(DEV), None, 0.5,
                           state, slots, cu, out, H, H, dk, dv, parts=parts)
        results.append((out.cpu(), state.cpu()))
    # the oracle, with the start states
    at = 0
    for i, n in enumerate(lens):
        S = start[i].reshape(H, dk, dv).clone()
        want = torch.zeros(n, H, dv, dtype=torch.float64)
        qq, kk, vv, aa = (x[at:at + n].reshape(n, H, -1) for x in (q, k, v, a))
        for t in range(n):
            S = aa[t][:, :, None] * S + kk[t][:, :, None] * vv[t][:, None, :]
            want[t] = torch.einsum("hkv,hk->hv", S, qq[t] * 0.5)
        for out, state in results:
            np.testing.assert_allclose(out[at:at + n].numpy(), want.reshape(n, -1).numpy(), atol=3e-4 * float(want.abs().max()), rtol=3e-4)
            np.testing.assert_allclose(state[int(slots[i])].numpy(), S.reshape(-1).numpy(), atol=3e-4 * float(S.abs().max()), rtol=3e-4)
        at += n
    assert all(torch.equal(st[3], torch.zeros(H * dk * dv)) for _, st in results)


@pytest.mark.parametrize("rule", ["gla", "delta"])
def test_recurrence_inputs_as_odd_column_ranges(rule):
    """q, k, decays, v and beta as ranges of columns that start at odd offsets of rows of odd length (no 16-byte copies),
    with a portion long enough to be cut into parts."""
    from boring_llm_b200.kernels import ops
    H, G, dk, dv, T = 2, (2 if rule == "gla" else 1), 32, 24, 300
    wide = lambda cols, seed, scale=1.0: (rnd(T, cols + 7, seed=seed, scale=scale).float().to(DEV))[:, 3:3 + cols]
    q, k, v, beta = wide(G * dk, 1, 0.4), wide(G * dk, 2, 0.4), wide(H * dv, 3), wide(H, 4)
    a = (torch.rand(T, H * dk + 5, generator=torch.Generator().manual_seed(5)) * 0.1 + 0.9).to(DEV)[:, 1:1 + H * dk]
    assert q.stride(0) % 4 != 0 and a.data_ptr() % 16 != 0
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    slots = torch.tensor([1], dtype=torch.int32, device=DEV)
    outs = []
    for parts in (1, 7):
        state = torch.zeros(2, H * dk * dv, device=DEV)
        out = torch.empty(T, H * dv, device=DEV)
        ops.recurrent_scan(ops.RULE_GLA if rule == "gla" else ops.RULE_DELTA, q, k, v, a, beta if rule == "delta" else None, 1.0,
                           state, slots, cu, out, H, G, dk, dv, parts=parts)
        outs.append(out.cpu())
    d = lambda x, h, w: x.cpu().double().reshape(T, h, w)
    if rule == "gla":
        want = pf.gated_linear_recurrence(d(q, H, dk), d(k, H, dk), d(v, H, dv), d(a, H, dk))
    else:
        want = pf.delta_recurrence(d(q, G, dk).repeat_interleave(H // G, 1), d(k, G, dk).repeat_interleave(H // G, 1), d(v, H, dv),
                                   d(a, H, dk), torch.sigmoid(beta.cpu().double()))
    for out in outs:
        np.testing.assert_allclose(out.numpy(), want.reshape(T, -1).numpy(), atol=3e-4 * float(want.abs().max()), rtol=3e-4)


@pytest.mark.parametrize("H,G,dk,dv", [(2, 1, 16, 24), (1, 1, 64, 40), (3, 3, 48, 8), (2, 2, 128, 32)])
def test_long_portions_of_the_delta_rule_cut_into_parts(H, G, dk, dv):
    """As for linear attention, with the delta rule's transition over a part as a matrix: the walk in one piece, 16 parts
    and 5 parts against the oracle, from states an earlier step left; a short request in the same step is not cut."""
    from boring_llm_b200.kernels import ops
    lens = [600, 300, 30]
    T = sum(lens)
    q, k = rnd(T, G, dk, seed=1, scale=0.5), rnd(T, G, dk, seed=2)
    k = k / k.norm(dim=-1, keepdim=True)
    v, beta = rnd(T, H, dv, seed=3), rnd(T, H, seed=6)
    a = torch.rand(T, H, dk, generator=torch.Generator().manual_seed(4), dtype=torch.float64) * 0.08 + 0.92
    start = rnd(3, H, dk, dv, seed=5)
    cu = torch.tensor(np.cumsum([0] + lens), dtype=torch.int32, device=DEV)
    slots = torch.tensor([2, 0, 1], dtype=torch.int32, device=DEV)
    f = lambda x: x.reshape(T, -1).float().to(DEV).contiguous()
    results = []
    for parts in (1, ops.SCAN_MAX_PARTS, 5):
        state = torch.zeros(4, H * dk * dv + 3, device=DEV)
        state[slots.long(), :H * dk * dv] = start.reshape(3, -1).float().to(DEV)
        out = torch.empty(T, H * dv, device=DEV)
        ops.recurrent_scan(ops.RULE_DELTA, f(q), f(k), f(v), f(a), f(beta), 0.5, state, slots, cu, out, H, G, dk, dv, parts=parts)
        results.append((out.cpu(), state.cpu()))
    rep = H // G
    at = 0
    for i, n in enumerate(lens):
        S = start[i].clone()
        want = torch.zeros(n, H, dv, dtype=torch.float64)
        for t in range(at, at + n):
            kk, qq = k[t].repeat_interleave(rep, 0), q[t].repeat_interleave(rep, 0) * 0.5
            S = a[t][:, :, None] * S
            u = torch.sigmoid(beta[t])[:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, kk))
            S = S + kk[:, :, None] * u[:, None, :]
            want[t - at] = torch.einsum("hkv,hk->hv", S, qq)
        for out, state in results:
            np.testing.assert_allclose(out[at:at + n].numpy(), want.reshape(n, -1).numpy(), atol=5e-4 * float(want.abs().max()), rtol=5e-4)
            np.testing.assert_allclose(state[int(slots[i]), :H * dk * dv].numpy(), S.reshape(-1).numpy(), atol=5e-4 * float(S.abs().max()), rtol=5e-4)
        at += n
    assert all(torch.equal(st[3], torch.zeros(H * dk * dv + 3)) and torch.equal(st[:, H * dk * dv:], torch.zeros(4, 3)) for _, st in results)
