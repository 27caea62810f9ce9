"""The Kavotar decoder on the GPU against the plain float64 implementation in `plain_kavotar`: each mechanism alone
through its kernels, then whole models of several small shapes through the runner (prompts whole, tails token by token,
portions down to two tokens, mixed batches with pages and slots used again), and greedy generation through `Engine`.
The test models are random; where random weights would hide a fault the inputs are made so that it shows."""
import numpy as np
import pytest
import torch

import helpers
import plain_kavotar as pk
import plain_model as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


# ---- small shapes -----------------------------------------------------------------------------------------------------
def memory(heads, dim, vdim, cap):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def parallel(heads, kv, dim, vdim, chunk, rot, base, scale, r_heads, r_dim, rank):
    return {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": chunk}, "rot": {"base": base, "dims": rot},
                 "scale": scale},
        "right": {"heads": r_heads, "dim": r_dim, "rank": rank}}}


def with_moe(layer, ff, experts, top, count, keep):
    return dict(layer, mlp={"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top,
                                                                           "groups": {"count": count, "keep": keep}}})


def bare(layer):
    return dict(layer, mlp=None)


SHAPES = {
    # both mixers, values wider and narrower than keys, a chunk that is no multiple of the page, groups of which two stay
    "A": {"architecture": "Kavotar", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 9.0, "layers": [
        with_moe(memory(2, 24, 16, 6.0), 40, 8, 2, 4, 2),
        with_moe(parallel(4, 2, 16, 24, 20, 8, 10000.0, 0.3, 2, 16, 8), 32, 6, 3, 3, 2),
        bare(memory(3, 8, 24, 15.0)),
        with_moe(parallel(2, 1, 32, 16, 37, 32, 500000.0, 0.2, 4, 8, 4), 48, 4, 1, 1, 1)]},
    # sizes that are 1 or equal: one head everywhere, chunks of one position (a token sees itself only) and of two, one
    # expert a token out of two, groups of one expert each
    "B": {"architecture": "Kavotar", "vocab": 61, "width": 40, "norm": {"eps": 1e-6}, "logit_softcap": 30.0, "layers": [
        with_moe(parallel(1, 1, 8, 8, 1, 2, 100.0, 1.0, 1, 8, 2), 40, 2, 1, 2, 1),
        with_moe(memory(1, 8, 8, 1.0), 16, 1, 1, 1, 1),
        with_moe(parallel(1, 1, 16, 8, 2, 0, 100.0, 0.5, 1, 16, 16), 24, 4, 2, 4, 2)]},
    # nothing is a multiple of 4, every head its own key/value head, rotation of a part of the head
    "C": {"architecture": "Kavotar", "vocab": 77, "width": 50, "norm": {"eps": 1e-6}, "logit_softcap": 12.0, "layers": [
        with_moe(parallel(3, 3, 10, 6, 33, 6, 50.0, 0.3, 2, 9, 5), 30, 5, 2, 1, 1),
        with_moe(memory(2, 20, 9, 4.0), 22, 9, 4, 3, 2)]},
    # no attention at all (no pages, only state slots)
    "D": {"architecture": "Kavotar", "vocab": 83, "width": 48, "norm": {"eps": 1e-5}, "logit_softcap": 20.0, "layers": [
        with_moe(memory(2, 16, 16, 8.0), 64, 4, 2, 2, 1),
        bare(memory(3, 16, 8, 8.0))]},
    # wider rows and head size 64: prompts of a few hundred tokens send the products through the tcgen05 kernels
    "E": {"architecture": "Kavotar", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "logit_softcap": 15.0, "layers": [
        with_moe(parallel(6, 2, 64, 64, 150, 32, 500000.0, 0.11, 4, 32, 16), 128, 8, 2, 2, 1),
        with_moe(memory(4, 32, 64, 10.0), 64, 16, 4, 4, 2)]},
}
# every open expert is taken (two of two): no choice that rounding could turn
SHAPES["F"] = {"architecture": "Kavotar", "vocab": 77, "width": 48, "norm": {"eps": 1e-6}, "logit_softcap": 12.0, "layers": [
    with_moe(parallel(4, 2, 16, 8, 12, 8, 1000.0, 0.25, 2, 16, 4), 32, 2, 2, 1, 1),
    with_moe(memory(2, 16, 24, 5.0), 24, 2, 2, 1, 1)]}
SEEDS = {"A": 21, "B": 22, "C": 23, "D": 24, "E": 25, "F": 26}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from boring_llm_b200 import KavotarConfig, write_random_model
    made = {}

    def get(name, std=0.25):
        key = (name, std)
        if key not in made:
            d = str(tmp_path_factory.mktemp(f"kav_{name}"))
            write_random_model(d, KavotarConfig.from_dict(SHAPES[name]), SEEDS[name], "bfloat16", std)
            made[key] = d
        return made[key]
    return get


def plain_logits(folder, tokens):
    cfg, W = plain.read_model_folder(folder)
    return pk.forward(cfg, W, tokens).numpy()


def run_recording(folder, dtype, steps, max_tokens, debug_poison=False):
    """`helpers.run_inprocess` with kernels launched singly, which also returns the experts every feed-forward chose:
    {layer: {(request, position): experts}}."""
    from boring_llm_b200.config import EngineOptions
    from boring_llm_b200.engine.runner import ModelRunner, StepEntry
    from boring_llm_b200.models import load_model
    cfg, model = load_model(folder, dtype, DEV)
    cap = -(-max_tokens // 16) * 16
    runner = ModelRunner(model, EngineOptions(dtype=dtype, page_size=16, max_tokens=cap, ctx_size=cap, max_num_seqs=8,
                                              cuda_graphs=False, debug_poison=debug_poison))
    moe = {i: b.ffn for i, b in enumerate(model.blocks) if b.ffn is not None}
    for part in moe.values():
        part.record = []
    outputs, chosen, at = {}, {i: {} for i in moe}, {}
    for s in steps:
        logits = runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]])
        if logits.shape[0]:
            outputs[s["step"]] = logits.float().cpu().numpy()
        for i, part in moe.items():
            ids = part.record.pop().cpu()
            assert not part.record
            t = 0
            for e in s["entries"]:
                for j in range(len(e["tokens"])):
                    chosen[i][(e["id"], at.get(e["id"], 0) + j)] = ids[t]
                    t += 1
        for e in s["entries"]:
            at[e["id"]] = at.get(e["id"], 0) + len(e["tokens"])
        for rid in s["end"]:
            runner.free_request(rid)
            at.pop(rid, None)
    runner.cache.check()
    return outputs, runner, chosen


def check_trace(folder, dtype, reqs, steps, max_tokens, what, tol=None, **kw):
    """float32: the engine against the plain implementation, experts and all. bfloat16: rounding may turn a close choice
    between two experts the other way, so the plain implementation is told which experts the engine took, and the
    engine's choice must be the plain one wherever that is not close."""
    if dtype == "float32":
        outputs, runner = helpers.run_inprocess(folder, dtype, steps, max_tokens, **kw)
        chosen = None
    else:
        outputs, runner, chosen = run_recording(folder, dtype, steps, max_tokens, **kw)
    rows = helpers.collect_rows(steps, outputs)
    cfg, W = plain.read_model_folder(folder)
    errors, scale = [], 1e-6
    for rid, toks in reqs.items():
        forced = None if chosen is None else {i: torch.stack([c[(rid, p)] for p in range(len(toks))]) for i, c in chosen.items()}
        info = {}
        want = pk.forward(cfg, W, toks, forced=forced, info=info).numpy()
        got = np.stack([rows[(rid, p)] for p in range(len(toks))])
        assert np.isfinite(got).all(), f"{what} {rid}: non-finite logits"
        if dtype == "float32":
            helpers.assert_close(got, want, dtype, f"{what} {rid}")
            continue
        errors.append(np.abs(got - want).max(-1))
        scale = max(scale, np.abs(want).max())
        for i, (own, margin) in info.items():
            same = (own.sort(-1).values == forced[i].long().sort(-1).values).all(-1)
            assert bool((same | (margin < 0.05)).all()), f"{what} {rid}: layer {i} chose other experts where the choice is clear"
    if errors:
        # The design has places where rounding is amplified without bound (the first tokens of a matrix memory: a read-out
        # k . q that happens to cancel, times the exponential of an input gate; a norm behind a sublayer whose result is
        # small), so a few positions of a random model may lie far off in bfloat16. A fault of the engine moves most
        # positions; the 32-bit runs of the same traces hold every position to 1e-4.
        e = np.concatenate(errors) / scale
        over = int((e > tol).sum())
        assert over <= max(1, int(0.04 * e.size)), f"{what}: {over} of {e.size} positions differ by more than {tol} (worst {e.max():.3f})"
        assert np.median(e) <= tol / 4, f"{what}: median difference {np.median(e):.4f}"
    return runner


def solo_steps(reqs, cut):
    steps, n0 = [], 0
    for i, (rid, toks) in enumerate(reqs.items()):
        s = helpers.solo_trace(rid, toks, cut(toks, i), n0)
        steps += s
        n0 += len(s)
    return steps


# bfloat16 against pure float64: activations are rounded to 8 bits between kernels, and a token whose two best experts
# lie close may take the other one
BF16_TOL = 6e-2


def std_for(dtype):
    return 0.25 if dtype == "float32" else 0.1


# ---- whole models ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_whole_tails_singly_and_portions(folders, name, dtype):
    folder = folders(name, std_for(dtype))
    vocab = SHAPES[name]["vocab"]
    reqs = {f"r{i}": helpers.random_tokens(vocab, n, 100 + i) for i, n in enumerate([1, 2, 19, 75, 130])}
    tol = None if dtype == "float32" else BF16_TOL
    check_trace(folder, dtype, reqs, solo_steps(reqs, lambda t, i: helpers.cut_whole(t)), 256, f"{name} whole", tol)
    check_trace(folder, dtype, reqs, solo_steps(reqs, lambda t, i: helpers.cut_tail_singly(t, 45)), 256, f"{name} tail", tol)
    check_trace(folder, dtype, reqs, solo_steps(reqs, lambda t, i: helpers.cut_varying(t, i)), 256, f"{name} portions", tol)
    check_trace(folder, dtype, reqs, solo_steps(reqs, lambda t, i: [2] * (len(t) // 2) + [1] * (len(t) % 2)), 256,
                f"{name} pairs", tol)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_reuse_pages_and_slots(folders, name, dtype):
    folder = folders(name, std_for(dtype))
    vocab = SHAPES[name]["vocab"]
    reqs = {f"m{i}": helpers.random_tokens(vocab, n, 200 + i) for i, n in enumerate([33, 7, 90, 41, 2, 64, 17, 58])}
    steps, peak = helpers.mixed_trace(reqs, seed=5, max_live=3)
    runner = check_trace(folder, dtype, reqs, steps, peak, f"{name} mixed", None if dtype == "float32" else BF16_TOL,
                         debug_poison=True)
    assert all(hw <= runner.cache.num_pages for hw in runner.cache.stats()["pages_high_water"])
    assert len(runner.cache.state_groups) >= 1 and (len(runner.cache.paged_groups) >= 1) == (name != "D")


def test_float32_does_not_depend_on_the_cut_or_the_batch(folders):
    folder = folders("A")
    reqs = {f"c{i}": helpers.random_tokens(97, n, 300 + i) for i, n in enumerate([50, 21, 77])}
    a, _ = helpers.run_inprocess(folder, "float32", solo_steps(reqs, lambda t, i: helpers.cut_whole(t)), 256)
    whole = helpers.collect_rows(solo_steps(reqs, lambda t, i: helpers.cut_whole(t)), a)
    steps, peak = helpers.mixed_trace(reqs, seed=9, max_live=3)
    b, _ = helpers.run_inprocess(folder, "float32", steps, peak)
    mixed = helpers.collect_rows(steps, b)
    for key, row in whole.items():
        assert np.abs(row - mixed[key]).max() <= 2e-5 * max(1.0, np.abs(row).max()), key


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_many_chunk_edges(folders, dtype):
    folder = folders("A", std_for(dtype))
    toks = helpers.random_tokens(97, 330, 7)
    steps = helpers.solo_trace("long", toks, [30] + [1] * 300)
    runner = check_trace(folder, dtype, {"long": toks}, steps, 384, "long decoding", None if dtype == "float32" else BF16_TOL)
    # the pages before the current chunk went back while the request was running: it never held all of its 21 pages
    assert max(runner.cache.stats()["pages_high_water"]) <= 6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wide_shape_on_the_tensor_core_products(folders, dtype):
    """Prompts of 300 and 90 tokens: in bfloat16 the joined projections run on tcgen05, decode steps replay captured
    graphs; a chunk wider than a key block; a portion of more than 256 tokens is cut into parts by the scans."""
    folder = folders("E", 0.25 if dtype == "float32" else 0.06)
    reqs = {"w0": helpers.random_tokens(300, 300, 1), "w1": helpers.random_tokens(300, 90, 2)}
    tol = None if dtype == "float32" else BF16_TOL
    steps = solo_steps(reqs, lambda t, i: helpers.cut_tail_singly(t, 24))
    check_trace(folder, dtype, reqs, steps, 512, "wide tail", tol).check_kernels()
    steps, peak = helpers.mixed_trace(reqs, seed=3, max_live=2)
    check_trace(folder, dtype, reqs, steps, peak, "wide mixed", tol).check_kernels()


def test_captured_steps_replay_the_same_bits(folders):
    folder = folders("A", 0.1)
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
    for name, dtype, std in (("A", "float32", 0.25), ("C", "float32", 0.25), ("F", "bfloat16", 0.1)):
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


def test_layer_streams_one_by_one(folders):
    """float32: the residual stream behind every layer against the plain implementation's."""
    from boring_llm_b200.config import EngineOptions
    from boring_llm_b200.engine.runner import ModelRunner, StepEntry
    from boring_llm_b200.models import load_model
    folder = folders("A")
    toks = helpers.random_tokens(97, 70, 3)
    cfg, W = plain.read_model_folder(folder)
    _, want = pk.forward(cfg, W, toks, streams=True)
    _, model = load_model(folder, "float32", DEV)
    runner = ModelRunner(model, EngineOptions(dtype="float32", max_tokens=128, ctx_size=128, max_num_seqs=2, cuda_graphs=False))
    model.keep_streams = []
    runner.step([StepEntry("s", toks, [])])
    assert len(model.keep_streams) == len(cfg["layers"])
    for i, got in enumerate(model.keep_streams):
        w = want[i].numpy()
        assert np.abs(got.cpu().numpy() - w).max() <= 1e-4 * np.abs(w).max(), i


# ---- mechanisms alone --------------------------------------------------------------------------------------------------
def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float64) * scale


def dev(t, dtype=torch.float32):
    return t.to(dtype).to(DEV).contiguous()


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def paged(x, page, n_pages, order):
    """x [T, G, d] of one request -> (cache [n_pages + 1, G, page, d], NaN wherever the request holds nothing; block table row)."""
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


@pytest.mark.parametrize("H,G,dk,dv,chunk", [(4, 2, 16, 16, 40), (3, 1, 24, 8, 21), (2, 2, 8, 40, 16), (1, 1, 32, 32, 1), (6, 3, 16, 72, 150),
                                             (2, 1, 16, 16, 0)])
def test_chunk_attention_kernel_with_planted_keys(H, G, dk, dv, chunk):
    """Keys at chosen places get a score that dominates: the first and the last position of a chunk seen from the chunk's
    last and from the next chunk's first position, at page borders, the sequence's first token. Pages are scattered, the
    unused rest of the pool is NaN, the request arrives in two portions and then singly; the heads' weights are mixed."""
    from boring_llm_b200.kernels import ops
    T, page = 150, 16
    q, k, v = rnd(T, H, dk, seed=1), rnd(T, G, dk, seed=2), rnd(T, G, dv, seed=3)
    talk, temp = rnd(H, H, seed=4), rnd(H, seed=5).abs() + 0.5
    c = chunk or 1000
    pairs = [(149, 149 - 149 % c), (149, max(0, 149 - 149 % c - 1)), (2 * c - 1 if 2 * c - 1 < T else 100, c), (min(2 * c, T - 1), c),
             (min(2 * c, T - 1), min(2 * c, T - 1) - 1), (100, 96), (100, 95), (64, 63), (64, 48), (33, 32), (16, 15), (16, 0), (c - 1 if c - 1 < T else 5, 0)]
    for qi, kj in [(a, b) for a, b in pairs if b <= a < T]:
        k[kj] = k[kj] * 0 + q[qi, 0] / q[qi, 0].norm() * 6.0
    want = pk.talking_attention(q, k, v, 0.3, temp, talk, c)
    order = list(np.random.default_rng(0).permutation(12))
    kc, table = paged(k, page, 12, order)
    vc, _ = paged(v, page, 12, order)
    out = torch.empty(T, H * dv, device=DEV)
    tb = i32([table + [-1] * (16 - len(table))])
    at = 0
    for n in [90, 50] + [1] * 10:
        sl = slice(at, at + n)
        A = torch.empty(n, H, G, dv, device=DEV)
        ops.attention_talk_plain(dev(q[sl].reshape(n, H * dk)), kc.to(DEV), vc.to(DEV), torch.zeros(n, dtype=torch.int32, device=DEV),
                                 i32([0, n]), i32([at + n]), tb, A, H, chunk, 0, 0.3, dev(temp))
        o = torch.empty(n, H * dv, device=DEV)
        ops.talk_mix(A, dev(talk), o)
        out[sl] = o
        at += n
    got = out.cpu().numpy().reshape(T, H, dv)
    assert np.isfinite(got).all()
    np.testing.assert_allclose(got, want.numpy(), atol=5e-5, rtol=3e-4)
    # a key just outside the chunk must not be seen, one just inside must: moving the edge by one shows in the oracle
    if 1 < c < 100:
        other = pk.talking_attention(q, k, v, 0.3, temp, talk, c + 1)
        assert (other - want).abs().max() > 1e-2


@pytest.mark.parametrize("H,dk,dv", [(2, 24, 16), (3, 20, 9), (1, 64, 40), (2, 130, 8)])
def test_matrix_memory_kernels_in_portions_with_slots_used_again(H, dk, dv):
    """Two requests in one batch (unequal portions, one sitting a step out), states in slots that were left dirty and then
    cleared; forget gates near one, so the first token still counts after 230 steps; input gates large enough for the
    running maximum to move, and gate pre-activations beyond the cap."""
    from boring_llm_b200.kernels import ops
    lens = {"a": 230, "b": 57}
    cap, eps = 5.0, 1e-5
    data, want = {}, {}
    bi, bf = rnd(H, seed=3), rnd(H, seed=4) * 0.3 + 8.0
    norm_w = rnd(H * dv, seed=5) + 1.0
    for i, (rid, T) in enumerate(lens.items()):
        q, k, v = rnd(T, H, dk, seed=10 + i, scale=0.5), rnd(T, H, dk, seed=20 + i, scale=0.5), rnd(T, H, dv, seed=30 + i)
        zi, zf, g = rnd(T, H, seed=40 + i, scale=4.0), rnd(T, H, seed=50 + i, scale=1.0), rnd(T, H * dv, seed=60 + i)
        zi[0] = 10.0                              # the first token enters at the cap: later maxima cannot push it below e^(sum of f)
        data[rid] = (q, k, v, zi, zf, g)
        o = pk.matrix_memory(q * dk ** -0.5, k, v, pk.soft_cap(zi + bi, cap), pk.log_sigmoid(pk.soft_cap(zf + bf, cap)))
        want[rid] = (pk.rms_unit(o, eps).reshape(T, H * dv) * norm_w * torch.sigmoid(g)).numpy()
    n_s = H * dk * (dv + 1)                    # the normaliser is the state's last value column
    n_state = n_s + H
    state = torch.full((4, n_state + 5), float("nan"), device=DEV)
    slots = {"a": 2, "b": 0}
    for s in slots.values():
        state[s, :n_state].zero_()
    got = {rid: torch.zeros(T, H * dv) for rid, T in lens.items()}
    at = {"a": 0, "b": 0}
    off_k, off_v, off_g, off_i, off_f = H * dk, 2 * H * dk, 2 * H * dk + H * dv, 2 * H * dk + 2 * H * dv, 2 * H * dk + 2 * H * dv + H
    for step in [{"a": 100, "b": 2}, {"a": 1}, {"b": 30, "a": 64}, {"a": 2, "b": 1}, {"b": 24, "a": 63}]:
        rids = list(step)
        rows = []
        for r in rids:
            q, k, v, zi, zf, g = (t[at[r]:at[r] + step[r]] for t in data[r])
            n = step[r]
            rows.append(torch.cat([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1), g, zi, zf], dim=1))
        proj = dev(torch.cat(rows))
        T = proj.shape[0]
        cu = i32(np.cumsum([0] + [step[r] for r in rids]))
        sl = i32([slots[r] for r in rids])
        decay, keys, values, floor = ops.memory_gates(proj, off_k, off_v, off_i, off_f, dev(bi), dev(bf), cap, state, n_s, sl, cu, H, dk, dv)
        o = torch.empty(T, H * (dv + 1), device=DEV)
        ops.recurrent_scan(ops.RULE_GLA, proj[:, :off_k], keys, values, decay, None, dk ** -0.5, state, sl, cu, o, H, H, dk, dv + 1)
        y = torch.empty(T, H * dv, device=DEV)
        ops.head_norm_gate_ext(o, dev(norm_w), proj[:, off_g:off_i], ops.GATE_SIGMOID, eps, y, H, dv, floor=floor)
        y = y.cpu()
        t0 = 0
        for r in rids:
            got[r][at[r]:at[r] + step[r]] = y[t0:t0 + step[r]]
            t0 += step[r]; at[r] += step[r]
    assert at == lens
    for rid in lens:
        np.testing.assert_allclose(got[rid].numpy(), want[rid], atol=3e-4 * max(1.0, np.abs(want[rid]).max()), rtol=3e-4)
    assert torch.isnan(state[1]).all() and torch.isnan(state[3]).all() and torch.isnan(state[0, n_state:]).all()
    # the first token still counts at the end of request a
    q, k, v, zi, zf, g = data["a"]
    v2 = v.clone(); v2[0] = 0
    i_log, f_log = pk.soft_cap(zi + bi, cap), pk.log_sigmoid(pk.soft_cap(zf + bf, cap))
    full, cut = pk.matrix_memory(q * dk ** -0.5, k, v, i_log, f_log)[-1], pk.matrix_memory(q * dk ** -0.5, k, v2, i_log, f_log)[-1]
    assert (full - cut).abs().max() > 1e-3 * full.abs().max()


@pytest.mark.parametrize("H,dk", [(2, 24), (3, 20), (1, 64), (2, 130)])
@pytest.mark.parametrize("long_parts", [1, 5])
def test_bonus_recurrence_with_token_shift_in_portions(H, dk, long_parts):
    """Token shift (the row before a step's first token comes from the slot), decays from their two factors, the bonus and
    the read-out before the write, two requests in dirty slots; with `long_parts` > 1 a portion of 300 tokens is cut into
    parts that run side by side."""
    from boring_llm_b200.kernels import ops
    d, rank = 40, 6
    lens = {"a": 330, "b": 57}
    mu = torch.rand(5, d, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    Wr, Wk, Wv = rnd(H * dk, d, seed=2, scale=0.2), rnd(H * dk, d, seed=3, scale=0.2), rnd(H * dk, d, seed=4, scale=0.2)
    W1, W2, w0 = rnd(rank, d, seed=5, scale=0.3), rnd(H * dk, rank, seed=6, scale=0.5), rnd(H * dk, seed=7, scale=0.5) - 4.0
    u = rnd(H, dk, seed=8)
    data, want = {}, {}
    for i, (rid, T) in enumerate(lens.items()):
        x = rnd(T, d, seed=10 + i)
        prev = torch.cat([torch.zeros(1, d, dtype=torch.float64), x[:-1]])
        mix = [x + (prev - x) * mu[s] for s in range(5)]
        r, k, v = (mix[0] @ Wr.T).view(T, H, dk), (mix[1] @ Wk.T).view(T, H, dk), (mix[2] @ Wv.T).view(T, H, dk)
        w = torch.exp(-torch.exp(torch.tanh(mix[4] @ W1.T) @ W2.T + w0)).view(T, H, dk)
        data[rid] = x
        want[rid] = pk.bonus_recurrence(r, k, v, w, u).reshape(T, H * dk).numpy()
    n_s = H * dk * dk
    state = torch.full((4, n_s + d + 3), float("nan"), device=DEV)
    slots = {"a": 3, "b": 1}
    for s in slots.values():
        state[s, :n_s + d].zero_()
    prev_rows = state[:, n_s:]
    got = {rid: torch.zeros(T, H * dk) for rid, T in lens.items()}
    at = {"a": 0, "b": 0}
    for step in [{"a": 300, "b": 2}, {"a": 1}, {"b": 30, "a": 2}, {"a": 1, "b": 1}, {"b": 24, "a": 26}]:
        rids = list(step)
        x = dev(torch.cat([data[r][at[r]:at[r] + step[r]] for r in rids]))
        T = x.shape[0]
        cu = i32(np.cumsum([0] + [step[r] for r in rids]))
        sl = i32([slots[r] for r in rids])
        tok_req = i32(np.repeat(np.arange(len(rids)), [step[r] for r in rids]))
        mixes = torch.empty(5, T, d, device=DEV)
        ops.shift_mix(x, dev(mu), prev_rows, sl, tok_req, cu, mixes)
        ops.conv_tail_update(x, 2, prev_rows, sl, cu, d)
        r, k, v, low = (torch.empty(T, n, device=DEV) for n in (H * dk, H * dk, H * dk, rank))
        for m, w, dst in ((0, Wr, r), (1, Wk, k), (2, Wv, v), (4, W1, low)):
            ops.gemm_plain(mixes[m], dev(w), dst)
        decay = torch.empty(T, H * dk, device=DEV)
        ops.gemm_plain_decay_exp(low, dev(W2), dev(w0), decay, x_tanh=True)
        bonus = torch.empty(T, H, device=DEV)
        ops.bonus_dot(r, k, dev(u), bonus, H, dk)
        o = torch.empty(T, H * dk, device=DEV)
        from boring_llm_b200.kernels import library
        parts = long_parts if library.load().bl_recurrent_scan_can_split(ops.RULE_BONUS, H, dk, dk) else 1
        ops.recurrent_scan(ops.RULE_BONUS, r, k, v, decay, bonus, 1.0, state, sl, cu, o, H, H, dk, dk, parts=parts)
        o = o.cpu()
        t0 = 0
        for rr in rids:
            got[rr][at[rr]:at[rr] + step[rr]] = o[t0:t0 + step[rr]]
            t0 += step[rr]; at[rr] += step[rr]
    assert at == lens
    for rid in lens:
        np.testing.assert_allclose(got[rid].numpy(), want[rid], atol=3e-4 * max(1.0, np.abs(want[rid]).max()), rtol=3e-4)
    assert torch.isnan(state[0]).all() and torch.isnan(state[2]).all() and torch.isnan(state[1, n_s + d:]).all()


def test_routing_with_groups_negative_scores_and_sizes_of_one():
    """Choice scores that are negative (a closed group must count as minus infinity, not as 0), corrections that change
    the choice but not the weights, groups of one expert, all groups kept, one expert."""
    from boring_llm_b200.kernels import ops
    T = 200
    for E, top, groups, keep, shift in ((12, 3, 4, 2, -3.0), (8, 2, 8, 3, 0.0), (6, 6, 2, 2, -1.5), (1, 1, 1, 1, 0.0), (16, 4, 2, 1, -2.0),
                                         (9, 2, 3, 1, 0.5)):
        z = rnd(T, E, seed=E, scale=2.0)
        corr = rnd(E, seed=E + 1) + shift
        idx, wt = pk.route_from_logits(z, corr, top, groups, keep)
        ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
        wts = torch.empty(T, top, device=DEV)
        ops.moe_route(dev(z), dev(corr), top, groups, keep, ids, wts)
        assert (ids.cpu().long() == idx).all(), (E, top, groups, keep)
        np.testing.assert_allclose(wts.cpu().numpy(), wt.numpy(), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_expert_products_and_their_weighted_sum(dtype):
    from boring_llm_b200.kernels import ops
    from boring_llm_b200.kernels.ops import EPI_SWIGLU
    T, d, ff, E, top = 37, 48, 20, 5, 3
    x = rnd(T, d, seed=1).to(dtype).double()
    Wg, Wu, Wd = (rnd(E, ff, d, seed=2, scale=0.3).to(dtype).double(), rnd(E, ff, d, seed=3, scale=0.3).to(dtype).double(),
                  rnd(E, d, ff, seed=4, scale=0.3).to(dtype).double())
    g = torch.Generator().manual_seed(5)
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)])
    wts = torch.rand(T, top, generator=g, dtype=torch.float64)
    want = torch.zeros(T, d, dtype=torch.float64)
    for t in range(T):
        for j in range(top):
            e = int(ids[t, j])
            want[t] += wts[t, j] * ((pk.silu(x[t] @ Wg[e].T) * (x[t] @ Wu[e].T)) @ Wd[e].T)
    act = torch.empty(T * top, ff, dtype=dtype, device=DEV)
    idd = ids.to(torch.int32).to(DEV).contiguous()
    ops.expert_gemm_plain(dev(x, dtype), top, dev(torch.cat([Wg, Wu], dim=1), dtype), idd, act, EPI_SWIGLU)
    y = torch.empty(T * top, d, device=DEV)
    ops.expert_gemm_plain(act, 1, dev(Wd, dtype), idd, y)
    out = torch.full((T, d), 2.0, device=DEV)
    ops.moe_combine(y, dev(wts), out, add=True)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    np.testing.assert_allclose(out.cpu().numpy() - 2.0, want.numpy(), atol=tol * want.abs().max(), rtol=tol)


def test_norm_behind_the_sublayer_pair_mean_cast_and_soft_cap():
    from boring_llm_b200.kernels import ops
    for rows, d in ((7, 40), (130, 50), (3, 256), (5, 4100)):
        x, a, b = rnd(rows, d, seed=1), rnd(rows, d, seed=2, scale=3.0), rnd(rows, d, seed=3, scale=0.1)
        w, wa, wb = rnd(d, seed=4) + 1, rnd(d, seed=5) + 1, rnd(d, seed=6) + 1
        xs = dev(x)
        y = torch.empty(rows, d, dtype=torch.bfloat16, device=DEV)
        ops.post_norm_residual(xs, dev(a), dev(w), 1e-5, y)
        want = x + pk.layer_norm(a, w, 1e-5)
        np.testing.assert_allclose(xs.cpu().numpy(), want.numpy(), atol=2e-5, rtol=1e-5)
        assert torch.equal(y, xs.to(torch.bfloat16))
        xs = dev(x)
        ops.post_norm_residual(xs, dev(a), dev(w), 1e-5, None, b=dev(b), wa=dev(wa), wb=dev(wb), rms_eps=1e-3)
        s = 0.5 * (pk.rms_unit(a, 1e-3) * wa + pk.rms_unit(b, 1e-3) * wb)
        np.testing.assert_allclose(xs.cpu().numpy(), (x + pk.layer_norm(s, w, 1e-5)).numpy(), atol=2e-5, rtol=1e-5)
        m = torch.empty(rows, d, device=DEV)
        ops.pair_rms_mean(dev(a), dev(wa), dev(b), dev(wb), 1e-3, m)
        np.testing.assert_allclose(m.cpu().numpy(), s.numpy(), atol=2e-5, rtol=1e-5)
        c = dev(a * 10)
        ops.softcap(c, 7.0)
        np.testing.assert_allclose(c.cpu().numpy(), pk.soft_cap(a * 10, 7.0).numpy(), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("H,G,dk,dv,rot,layout", [(4, 2, 16, 8, 16, 0), (3, 1, 12, 20, 6, 0), (2, 2, 8, 8, 0, 0), (2, 1, 16, 16, 8, 1)])
def test_norm_per_head_rotation_and_cache_write(H, G, dk, dv, rot, layout):
    from boring_llm_b200.kernels import ops
    from boring_llm_b200.parts import RotaryTable
    T, page, base, eps = 40, 16, 100.0, 1e-5
    proj = rnd(T, (H + G) * dk + G * dv + 3, seed=1)
    qw, kw = rnd(dk, seed=2) + 1, rnd(dk, seed=3) + 1
    positions = torch.arange(5, 5 + T)
    q = pk.rms_unit(proj[:, :H * dk].view(T, H, dk), eps) * qw
    k = pk.rms_unit(proj[:, H * dk:(H + G) * dk].view(T, G, dk), eps) * kw
    if layout == 0:
        q, k = pk.rotate_halves(q, positions, base, rot), pk.rotate_halves(k, positions, base, rot)
    else:
        import plain_fezopel as pf
        q, k = pf.rotate_interleaved(q, positions, base, rot), pf.rotate_interleaved(k, positions, base, rot)
    table = RotaryTable(dk, base, n_rot=rot, pairs="halves" if layout == 0 else "interleaved").to(DEV)
    q_out = torch.empty(T, H * dk, device=DEV)
    kc = torch.full((5, G, page, dk), float("nan"), device=DEV)
    vc = torch.full((5, G, page, dv), float("nan"), device=DEV)
    tb = i32([[3, 0, 2, 1]])
    factor = rnd(H, seed=9)                            # a factor per head on q, of either sign
    ops.qk_head_norm_rope_write(dev(proj), H * dk, (H + G) * dk, dev(qw), dev(kw), eps, positions.to(torch.int32).to(DEV),
                                torch.zeros(T, dtype=torch.int32, device=DEV), tb, table.inv_freq, table.rot_half, table.pair_layout,
                                q_out, kc, vc, H, G, dk, dv, q_head_scale=dev(factor))
    np.testing.assert_allclose(q_out.cpu().numpy().reshape(T, H, dk), (q * factor[None, :, None]).numpy(), atol=3e-5, rtol=1e-4)
    pages = [3, 0, 2, 1]
    for t in range(T):
        p = 5 + t
        np.testing.assert_allclose(kc[pages[p // page], :, p % page].cpu().numpy(), k[t].numpy(), atol=3e-5, rtol=1e-4)
        np.testing.assert_allclose(vc[pages[p // page], :, p % page].cpu().numpy(),
                                   proj[t, (H + G) * dk:(H + G) * dk + G * dv].view(G, dv).numpy(), atol=1e-6)


@pytest.mark.parametrize("dh,H,G,chunk", [(64, 4, 2, 40), (32, 6, 3, 150), (128, 2, 1, 16), (16, 2, 2, 0), (48, 3, 1, 100)])
def test_chunk_attention_on_tensor_cores(dh, H, G, chunk):
    """The two tensor-core shapes (tiles of 64 new tokens; single tokens with their keys cut into slices) against the
    plain implementation on the same bfloat16 values: planted keys at the chunks' edges, two requests in the batch, one of
    them decoding, scattered pages with NaN elsewhere."""
    from boring_llm_b200.kernels import ops
    from boring_llm_b200.parts.attention import attention_plan
    T, page = 300, 16
    bf = lambda t: t.to(torch.bfloat16).double()
    q, k, v = bf(rnd(T, H, dh, seed=1)), bf(rnd(T, G, dh, seed=2)), bf(rnd(T, G, dh, seed=3))
    talk = rnd(H, H, seed=4)
    c = chunk or 1000
    for qi in (299, 290, 2 * c if 2 * c < T else 150, 2 * c - 1 if 0 < 2 * c - 1 < T else 100, 64, 63):
        for kj in (qi - qi % c, max(0, qi - qi % c - 1)):
            k[kj] = bf(k[kj] * 0 + q[qi, 0] / q[qi, 0].norm() * 5.0)
    want = pk.talking_attention(q, k, v, 0.25, torch.ones(H, dtype=torch.float64), talk, c).numpy()
    # a second request of 40 tokens that decodes its 41st beside every step of the first
    q2, k2, v2 = bf(rnd(41, H, dh, seed=5)), bf(rnd(41, G, dh, seed=6)), bf(rnd(41, G, dh, seed=7))
    want2 = pk.talking_attention(q2, k2, v2, 0.25, torch.ones(H, dtype=torch.float64), talk, c).numpy()[40]
    order = list(np.random.default_rng(1).permutation(24))
    kc = torch.full((25, G, page, dh), float("nan"), dtype=torch.bfloat16, device=DEV)
    vc = torch.full((25, G, page, dh), float("nan"), dtype=torch.bfloat16, device=DEV)
    t1, t2 = order[:19], order[19:22]
    for tab, kk, vv in ((t1, k, v), (t2, k2, v2)):
        for i in range(kk.shape[0]):
            kc[tab[i // page], :, i % page] = kk[i].to(torch.bfloat16).to(DEV)
            vc[tab[i // page], :, i % page] = vv[i].to(torch.bfloat16).to(DEV)
    tb = i32([t1 + [-1] * 5, t2 + [-1] * 21])
    got = np.zeros((T, H, dh))
    at = 0
    for n, splits in ((200, 1), (90, 1), (1, 1), (1, 3), (1, 2), (1, 1), (1, 4), (1, 1), (1, 1), (1, 2), (1, 1), (1, 1)):
        q_lens, ctx_lens = [n, 1], [at + n, 41]
        plan = attention_plan(q_lens, ctx_lens)
        qq = torch.cat([q[at:at + n].reshape(n, H * dh), q2[40:41].reshape(1, H * dh)]).to(torch.bfloat16).to(DEV).contiguous()
        spread = torch.full((n + 1, H, G, dh), float("nan"), dtype=torch.bfloat16, device=DEV)
        cu, ctx = i32([0, n, n + 1]), i32(ctx_lens)
        tiles, singles = (torch.from_numpy(plan.arrays[a]).to(DEV) for a in ("tiles64", "singles"))
        if tiles.shape[0]:
            ops.attention_prefill_talk(qq, kc, vc, cu, ctx, tb, tiles, spread, H, chunk, 0, 0.25, None)
        ops.attention_decode_talk(qq, kc, vc, cu, ctx, tb, singles, splits, spread, H, chunk, 0, 0.25, None)
        out = torch.empty(n + 1, H * dh, dtype=torch.bfloat16, device=DEV)
        ops.talk_mix(spread, dev(talk), out)
        o = out.float().cpu().numpy().reshape(n + 1, H, dh)
        assert np.isfinite(o).all()
        got[at:at + n] = o[:n]
        np.testing.assert_allclose(o[n], want2, atol=3e-2 * np.abs(want2).max(), rtol=3e-2)
        at += n
    np.testing.assert_allclose(got, want, atol=3e-2 * np.abs(want).max(), rtol=3e-2)


def test_the_command_line_and_the_trace_program_on_a_model_folder(folders, tmp_path):
    """`bin/boring-llm` generates what the plain implementation's arg-max gives, and `bin/trace_run`, started as a user
    would start it, writes the logits of a mixed trace (float32)."""
    import os
    import subprocess
    import sys
    folder = folders("A")
    exe = [sys.executable, os.path.join(helpers.ROOT, "bin", "boring-llm")]
    prompt = helpers.random_tokens(97, 9, 3)
    p = subprocess.run(exe + ["--model", folder, "--prompt-tokens", ",".join(map(str, prompt)), "--n-predict", "6", "--dtype", "f32",
                              "--ctx-size", "64", "--ignore-eos"], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr
    toks = list(prompt)
    for _ in range(6):
        toks.append(int(plain_logits(folder, toks)[-1].argmax()))
    assert p.stdout.strip().splitlines()[-1] == "generated: " + ",".join(map(str, toks[9:]))
    reqs = {f"t{i}": helpers.random_tokens(97, n, 600 + i) for i, n in enumerate([30, 12, 45])}
    steps, peak = helpers.mixed_trace(reqs, seed=2, max_live=2)
    outputs = helpers.run_trace_program(folder, "float32", steps, peak, str(tmp_path / "out"), 97)
    rows = helpers.collect_rows(steps, outputs)
    for rid, t in reqs.items():
        helpers.assert_close(np.stack([rows[(rid, i)] for i in range(len(t))]), plain_logits(folder, t), "float32", rid)
