"""Kavotar without a GPU: configuration keys and errors, declared tensors, caches of a block that keeps two, pages given
back behind a chunk, and the plain implementation against closed forms."""
import copy
import math

import pytest
import torch

import plain_kavotar as pk
from boring_llm_b200 import ConfigError, KavotarConfig
from boring_llm_b200.cache import CacheManager, PagedKVSpec, StateSpec
from boring_llm_b200.models import build_model

CFG = {"architecture": "Kavotar", "vocab": 90, "width": 32, "norm": {"eps": 1e-5}, "logit_softcap": 8.0, "layers": [
    {"type": "mlstm", "mixer": {"heads": 2, "dim": 8, "vdim": 12, "gate_cap": 7.0},
     "mlp": {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}}},
    {"type": "parallel", "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 4, "mask": {"size": 24},
                                            "rot": {"base": 1000.0, "dims": 4}, "scale": 0.5},
                                   "right": {"heads": 2, "dim": 8, "rank": 3}}, "mlp": None}]}


def test_config_round_trip_and_fields():
    cfg = KavotarConfig.from_dict(CFG)
    assert cfg.to_dict() == KavotarConfig.from_dict(cfg.to_dict()).to_dict()
    assert cfg.logit_softcap == 8.0 and cfg.layers[0].mixer.gate_cap == 7.0 and cfg.layers[0].mlp.keep == 2
    left = cfg.layers[1].mixer.left
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.chunk, left.rot_dims, left.scale) == (4, 2, 8, 4, 24, 4, 0.5)
    assert cfg.layers[1].mlp is None and cfg.layers[1].mixer.right.rank == 3


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "lstm", "unknown layer type"),
    (("layers", 0, "mixer", "gate_cap"), 0.0, "gate_cap"),
    (("layers", 1, "mixer", "left", "kv_heads"), 3, "cannot share"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 5, "rot.dims"),
    (("layers", 0, "mlp", "router", "top"), 5, "can be chosen"),
    (("layers", 0, "mlp", "router", "groups", "count"), 4, "groups"),
    (("layers", 0, "mlp", "kind"), "dense", "not supported"),
    (("norm", "eps"), 0.0, "norm.eps"),
])
def test_config_errors_name_the_key(path, value, word):
    d = copy.deepcopy(CFG)
    at = d
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        KavotarConfig.from_dict(d)


def test_declared_tensors_and_caches():
    model = build_model(KavotarConfig.from_dict(CFG))
    specs = model.tensor_specs()
    for name, shape in {"embed": (90, 32), "head": (90, 32), "final.norm": (32,), "l0.norm1": (32,), "l0.mix.q": (16, 32),
                        "l0.mix.v": (24, 32), "l0.mix.i": (2, 32), "l0.mix.f.b": (2,), "l0.mix.norm": (24,), "l0.mlp.router": (6, 32),
                        "l0.mlp.correction": (6,), "l0.mlp.e5.down": (32, 24), "l1.mix.left.q": (32, 32), "l1.mix.left.k": (16, 32),
                        "l1.mix.left.v": (8, 32), "l1.mix.left.q.norm": (8,), "l1.mix.left.talk": (4, 4), "l1.mix.left.temp": (4,),
                        "l1.mix.left.o": (32, 16), "l1.mix.right.mu.w": (32,), "l1.mix.right.w1": (3, 32), "l1.mix.right.w2": (16, 3),
                        "l1.mix.right.u": (2, 8), "l1.mix.left.out": (32,), "l1.mix.right.out": (32,)}.items():
        assert tuple(specs[name].shape) == shape, name
    assert "l1.norm2" not in specs and "l1.mlp.router" not in specs
    # the parallel block keeps pages AND a state slot: two cache layers for one entry of the run order
    assert [c.cache for c in model.schedule] == [0, (1, 2)]
    caches = model.cache_specs()
    assert caches[0] == StateSpec((2 * 8 * 12 + 2 * 8 + 2,), "float32")
    assert caches[1] == PagedKVSpec(2, 8, 0, 4, 24) and caches[2] == StateSpec((2 * 8 * 8 + 32,), "float32")


def test_pages_behind_the_chunk_go_back():
    m = CacheManager([PagedKVSpec(1, 8, chunk=40), PagedKVSpec(1, 8)], page_size=16, capacity_tokens=160, max_requests=2)
    m.add_request("a")
    held = lambda g: sum(1 for p in m.get("a").tables[g] if p >= 0)
    for n, want in ((39, 3), (1, 1), (39, 3), (1, 0), (40, 1)):        # 39 -> 40 (chunk 1 starts: pages 0, 1 dead) -> 79 -> 80 (all five dead) -> 120
        assert m.reserve("a", n)
        m.commit("a", n)
        assert held(0) == want, (m.get("a").num_tokens, m.get("a").tables[0])
    assert held(1) == 8                         # the group without a chunk keeps everything
    m.free("a")
    m.check()
    assert all(g.pool.num_free == g.pool.num_pages for g in m.paged_groups)
    assert PagedKVSpec(1, 8, chunk=40).first_needed(79) == 40 and PagedKVSpec(1, 8, window=10, chunk=40).first_needed(79) == 70


# ---- the plain implementation against closed forms -------------------------------------------------------------------------
def test_chunk_mask_counts_from_zero():
    m = pk.chunk_mask(7, 3)
    assert m[2].tolist() == [True, True, True, False, False, False, False]
    assert m[3].tolist() == [False, False, False, True, False, False, False]
    assert m[6].tolist() == [False, False, False, False, False, False, True]


def test_identity_talk_is_plain_attention_and_uniform_talk_averages_heads():
    T, H, G, d = 9, 4, 2, 6
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(T, n, d, generator=g, dtype=torch.float64) for n in (H, G, G))
    temp = torch.ones(H, dtype=torch.float64)
    plain = pk.talking_attention(q, k, v, 0.4, temp, torch.eye(H, dtype=torch.float64), 4)
    for i in range(T):
        lo = i - i % 4
        for h in range(H):
            w = torch.softmax((k[lo:i + 1, h // 2] @ q[i, h]) * 0.4, 0)
            assert torch.allclose(plain[i, h], w @ v[lo:i + 1, h // 2])
    # zero queries: uniform weights, so any talk matrix only scales by its row sum
    talk = torch.randn(H, H, generator=g, dtype=torch.float64)
    out = pk.talking_attention(q * 0, k, v, 0.4, temp, talk, 4)
    assert torch.allclose(out[5, 3], talk[3].sum() * v[4:6, 1].mean(0))


def test_matrix_memory_against_its_unrolled_sum():
    """Without the running maximum: S_t = sum_j exp(i_j + sum_(l > j) f_l) k_j v_j^T; the maximum only rescales numerator
    and denominator alike while |n . q| exceeds exp(-m)."""
    T, dk, dv = 6, 4, 3
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(T, 1, dk, generator=g, dtype=torch.float64), torch.randn(T, 1, dk, generator=g, dtype=torch.float64)
    v = torch.randn(T, 1, dv, generator=g, dtype=torch.float64)
    i_log = torch.randn(T, 1, generator=g, dtype=torch.float64) + 3.0
    f_log = -torch.rand(T, 1, generator=g, dtype=torch.float64)
    out = pk.matrix_memory(q, k, v, i_log, f_log)
    for t in range(T):
        w = torch.stack([torch.exp(i_log[j, 0] + f_log[j + 1:t + 1, 0].sum()) for j in range(t + 1)])
        S = torch.einsum("j,jk,jv->kv", w, k[:t + 1, 0], v[:t + 1, 0])
        n = torch.einsum("j,jk->k", w, k[:t + 1, 0])
        num = S.T @ q[t, 0]
        mm = 0.0
        for j in range(t + 1):
            mm = max(float(f_log[j, 0]) + mm, float(i_log[j, 0]))
        want = num * math.exp(-mm) / (max(abs(float(n @ q[t, 0])) * math.exp(-mm), math.exp(-mm)) + 1e-6)
        assert torch.allclose(out[t, 0], want, rtol=1e-9, atol=1e-12)


def test_bonus_recurrence_first_tokens():
    dk = 3
    r, k, w = (torch.rand(2, 1, dk, dtype=torch.float64) + 0.5 for _ in range(3))
    v = torch.rand(2, 1, dk, dtype=torch.float64)
    u = torch.rand(1, dk, dtype=torch.float64)
    o = pk.bonus_recurrence(r, k, v, w, u)
    assert torch.allclose(o[0, 0], (u[0] * k[0, 0] * r[0, 0]).sum() * v[0, 0])                      # an empty state: the bonus alone
    assert torch.allclose(o[1, 0], (k[0, 0] * r[1, 0]).sum() * v[0, 0] + (u[0] * k[1, 0] * r[1, 0]).sum() * v[1, 0])   # token 0 undecayed


def test_routing_closed_groups_are_minus_infinity():
    # group 1 holds the two largest single scores' sum; all choice scores are negative, so a closed group written as 0 would win
    z = torch.tensor([[-3.0, -2.5, -1.0, -1.2, -4.0, -0.9]], dtype=torch.float64)
    corr = torch.full((6,), -2.0, dtype=torch.float64)
    idx, wt = pk.route_from_logits(z, corr, 2, 3, 1)
    assert sorted(idx[0].tolist()) == [2, 3] and torch.allclose(wt[0], torch.sigmoid(z[0, idx[0]]))
    # the correction moves the choice, not the weights
    corr2 = corr.clone(); corr2[0] = 5.0; corr2[1] = 5.0
    idx2, wt2 = pk.route_from_logits(z, corr2, 2, 3, 1)
    assert sorted(idx2[0].tolist()) == [0, 1] and torch.allclose(wt2[0], torch.sigmoid(z[0, idx2[0]]))
