"""Fezopel without a GPU: its configuration and registry entry, the tensors its parts declare, shapes that only a
checkpoint gives, pages whose values differ in size from their keys, and the plain implementation checked against
closed forms that need no second implementation."""
import json
import math

import numpy as np
import pytest
import torch

import plain_fezopel as pf

CFG = {"architecture": "Fezopel", "vocab": 53, "width": 24, "norm": {"eps": 1e-5}, "layers": [
    {"type": "gla", "mixer": {"heads": 2, "dim": 6, "vdim": 4, "tau": 4.0}, "mlp": None},
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "mask": {"size": 9},
                                    "rot": {"base": 1000.0, "dims": 4}, "scale": 0.5}, "mlp": {"kind": "dense", "ff": 32}},
    {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 4, "vdim": 6, "conv": 3}, "mlp": None}]}


def test_config_reads_its_keys_and_round_trips():
    from boring_llm_b200 import FezopelConfig
    from boring_llm_b200.config import resolve_architecture
    arch = resolve_architecture(CFG)
    assert arch.config_cls is FezopelConfig
    cfg = FezopelConfig.from_dict(CFG)
    assert (cfg.vocab_size, cfg.width, cfg.norm_eps, len(cfg.layers)) == (53, 24, 1e-5, 3)
    a = cfg.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.rot_base, a.rot_dims, a.scale) == (4, 2, 8, 6, 9, 1000.0, 4, 0.5)
    assert cfg.layers[0].ff == 0 and cfg.layers[1].ff == 32 and cfg.layers[0].mixer.rank is None
    assert cfg.to_dict() == CFG
    assert FezopelConfig.from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("edit,word", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][0].update(type="mamba"), "mamba"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "share"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda c: c["layers"][1]["mlp"].update(kind="routed"), "routed"),
    (lambda c: c["layers"][0]["mixer"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][2]["mixer"].pop("conv"), "conv"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_config_errors_name_the_key(edit, word):
    from boring_llm_b200 import ConfigError, FezopelConfig
    c = json.loads(json.dumps(CFG))
    edit(c)
    with pytest.raises(ConfigError) as e:
        FezopelConfig.from_dict(c)
    assert word in str(e.value)


def test_declared_tensors_and_sizes_that_only_the_file_gives(tmp_path):
    from boring_llm_b200 import FezopelConfig, build_model, write_random_model
    from boring_llm_b200.weights import WeightsError, load_checkpoint, write_model_folder
    cfg = FezopelConfig.from_dict(CFG)
    specs = build_model(cfg).tensor_specs()
    assert specs["l0.mix.a1"].shape == (-1, 24) and specs["l0.mix.a2"].shape == (12, -1)
    assert specs["l1.mix.q.norm"].shape == (32,) and specs["l1.mix.k.norm"].shape == (16,) and specs["l1.mix.sink"].shape == (4,)
    assert specs["l1.mix.g"].shape == (4, 24) and specs["l1.mix.o"].shape == (24, 24) and specs["l1.mlp.up"].shape == (32, 24)
    assert specs["l2.mix.q.conv"].shape == (8, 3) and specs["l2.mix.v.conv"].shape == (24, 3) and specs["l2.mix.A_log"].shape == (4,)
    assert specs["l2.mix.dt_bias"].shape == (16,) and specs["l2.dwa"].shape == (4,) and specs["l0.dwa"].shape == (2,)
    assert "l0.norm2" not in specs and "l1.norm2b.b" in specs and "l0.rg1.b" in specs and "final.norm.b" in specs
    with pytest.raises(ValueError, match="only a checkpoint gives"):
        write_random_model(str(tmp_path / "no"), cfg, 0)
    # with the inner sizes named, a random model is written; a reader without them takes them from the file
    c = json.loads(json.dumps(CFG))
    c["layers"][0]["mixer"]["rank"] = 5
    c["layers"][2]["mixer"].update(rank=3, gate_rank=7)
    d = str(tmp_path / "yes")
    write_random_model(d, FezopelConfig.from_dict(c), 0)
    got = load_checkpoint(d, specs)
    assert got["l0.mix.a1"].shape == (5, 24) and got["l2.mix.g2"].shape == (24, 7)
    bad = dict(got)
    bad["l1.mix.sink"] = torch.zeros(5)
    write_model_folder(str(tmp_path / "bad"), c, bad)
    with pytest.raises(WeightsError, match="l1.mix.sink"):
        load_checkpoint(str(tmp_path / "bad"), specs)


def test_cache_groups_by_key_and_value_size_and_state_by_shape():
    from boring_llm_b200 import FezopelConfig, build_model
    from boring_llm_b200.cache import CacheManager, PagedKVSpec, StateSpec
    c = json.loads(json.dumps(CFG))
    c["layers"].append(json.loads(json.dumps(c["layers"][1])))
    c["layers"].append(json.loads(json.dumps(c["layers"][0])))
    specs = build_model(FezopelConfig.from_dict(c)).cache_specs()
    assert specs[1] == PagedKVSpec(2, 8, 9, 6) and specs[1].value_dim == 6 and PagedKVSpec(2, 8).value_dim == 8
    assert specs[0] == StateSpec((2 * 6 * 4,), "float32")
    assert specs[2] == StateSpec((4 * 4 * 6 + 2 * (2 * 2 * 4 + 4 * 6),), "float32")
    m = CacheManager(specs, 16, 64, 2)
    assert len(m.paged_groups) == 1 and m.paged_groups[0].cache_layers == [1, 3]
    assert [g.cache_layers for g in m.state_groups] == [[0, 4], [2]]
    # a window of nine gives pages back once every later query has passed them
    m.add_request("a"); assert m.reserve("a", 40); m.commit("a", 40)
    assert m.get("a").tables[0][:2] == [-1, -1] and m.get("a").tables[0][2] >= 0


# ---- the plain implementation against closed forms ----------------------------------------------------------------------
def rnd(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64)


def test_plain_rotation_keeps_lengths_and_relative_angles():
    x = rnd(5, 2, 8, seed=1)
    y = pf.rotate_interleaved(x, [3, 4, 5, 6, 7], 100.0, 4)
    np.testing.assert_allclose(y[..., 4:], x[..., 4:])
    np.testing.assert_allclose((y[..., :4] ** 2).sum(-1), (x[..., :4] ** 2).sum(-1))
    a = pf.rotate_interleaved(x[:1].repeat(2, 1, 1), [10, 13], 100.0, 8)
    b = pf.rotate_interleaved(x[:1].repeat(2, 1, 1), [0, 3], 100.0, 8)
    np.testing.assert_allclose((a[0] * a[1]).sum(), (b[0] * b[1]).sum())            # a dot product sees only the distance
    np.testing.assert_allclose(pf.rotate_interleaved(x, [0] * 5, 100.0, 8), x)


def test_plain_window_counts_the_query_itself():
    q, k = torch.ones(6, 1, 2, dtype=torch.float64), torch.ones(6, 1, 2, dtype=torch.float64)
    v = torch.arange(6, dtype=torch.float64).reshape(6, 1, 1)
    no_sink = torch.full((1,), -1e9, dtype=torch.float64)
    out = pf.sink_window_attention(q, k, v, 1.0, 3, no_sink)[:, 0, 0]
    np.testing.assert_allclose(out, [0, 0.5, 1, 2, 3, 4])                            # the mean of the last three positions
    out = pf.sink_window_attention(q, k, v, 1.0, 1, no_sink)[:, 0, 0]
    np.testing.assert_allclose(out, [0, 1, 2, 3, 4, 5])
    half = pf.sink_window_attention(q, k, v, 1.0, 1, torch.full((1,), 2.0, dtype=torch.float64))[:, 0, 0]
    np.testing.assert_allclose(half, np.arange(6) / 2)                                # a sink equal to the score halves it


def test_plain_recurrences_against_their_sums():
    T, H, dk, dv = 7, 2, 3, 4
    q, k, v, a = rnd(T, H, dk, seed=1), rnd(T, H, dk, seed=2), rnd(T, H, dv, seed=3), torch.rand(T, H, dk, dtype=torch.float64)
    o = pf.gated_linear_recurrence(q, k, v, a)
    for t in (0, 3, 6):
        want = torch.zeros(H, dv, dtype=torch.float64)
        for j in range(t + 1):
            w = (q[t] * k[j] * a[j + 1:t + 1].prod(0)).sum(-1)                        # decays of the steps after j
            want += w[:, None] * v[j]
        np.testing.assert_allclose(o[t], want, atol=1e-12)
    # delta rule: no decay, beta 1, orthonormal keys: reading with a key returns the value last written with it
    k = torch.eye(dk, dtype=torch.float64)[[0, 1, 2, 0, 1]].reshape(5, 1, dk)
    v = rnd(5, 1, dv, seed=4)
    o = pf.delta_recurrence(k, k, v, torch.ones(5, 1, dk, dtype=torch.float64), torch.ones(5, 1, dtype=torch.float64))
    np.testing.assert_allclose(o, v, atol=1e-12)                                     # the read-out sees the token's own write
    o = pf.delta_recurrence(k[[0, 0, 0, 0, 0]], k, v, torch.ones(5, 1, dk, dtype=torch.float64), torch.ones(5, 1, dtype=torch.float64))
    np.testing.assert_allclose(o[:, 0], torch.stack([v[0, 0], v[0, 0], v[0, 0], v[3, 0], v[3, 0]]), atol=1e-12)


def test_plain_convolution_is_causal_and_its_last_tap_is_now():
    x = rnd(6, 2, seed=1)
    w = torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]], dtype=torch.float64)
    y = pf.short_conv(x, w)
    np.testing.assert_allclose(y[:, 0], x[:, 0])
    np.testing.assert_allclose(y[:, 1], torch.cat([torch.zeros(2, dtype=torch.float64), x[:-2, 1]]))


def test_plain_layer_norm_and_forward_shapes():
    x = rnd(3, 10, seed=1) * 5 + 2
    y = pf.layer_norm(x, torch.ones(10, dtype=torch.float64), torch.zeros(10, dtype=torch.float64), 0.0)
    np.testing.assert_allclose(y.mean(-1), 0, atol=1e-12)
    np.testing.assert_allclose((y * y).mean(-1), 1, atol=1e-12)
    assert abs(float(pf.gelu_erf(torch.tensor(1.0, dtype=torch.float64))) - 0.5 * (1 + math.erf(1 / math.sqrt(2)))) < 1e-15


def test_command_line_lists_the_configuration_and_tensors(tmp_path, capsys):
    from boring_llm_b200 import FezopelConfig, write_random_model
    from boring_llm_b200 import cli
    c = json.loads(json.dumps(CFG))
    c["layers"][0]["mixer"]["rank"] = 5
    c["layers"][2]["mixer"].update(rank=3, gate_rank=7)
    d = str(tmp_path / "m")
    write_random_model(d, FezopelConfig.from_dict(c), 1)
    assert cli.main(["--model", d, "--dump-metadata"]) == 0
    out = capsys.readouterr().out
    assert "architecture = Fezopel" in out and "tensor l2.mix.q.conv [8, 3] matrix" in out and "tensor l0.dwa [2] norm" in out
