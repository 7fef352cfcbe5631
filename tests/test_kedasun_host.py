"""Host-side checks for the Kedasun family: the registry reads a model directory's config.json into the C structs, and the
plain restatement the GPU tests lean on is itself checked mechanism by mechanism on hand-made cases (no GPU)."""
import ctypes as C
import json
import math

import torch

from oracle import kedasun_oracle as O


def small_cfg():
    a = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "scale": 0.4, "rot": {"base": 50.0, "dims": 4}, "v_mix": True}
    b = {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 5, "scale": 0.3, "conv": 3, "mask": {"size": 5, "keep_first": 2}, "v_mix": True}
    mlp = {"kind": "dense", "ff": 14, "limit": 1.5}
    return {"architecture": "Kedasun", "vocab": 31, "width": 12, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5, "groups": 3}, "layers": [
        {"type": "attention", "mixer": a, "mlp": mlp}, {"type": "attention_2", "mixer": b, "mlp": None},
        {"type": "attention", "mixer": dict(a, v_mix=False), "mlp": mlp}]}


def test_registry_reads_the_layer_list(pkg, lib, tmp_path):
    from importlib import import_module
    capi = import_module("aws-k8s-ansible-provisioner_b200.capi")
    eng = import_module("aws-k8s-ansible-provisioner_b200.engine")
    cfg = small_cfg()
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    c = capi.b2_config()
    specs = (capi.b2_layer_spec * 8)()
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 8) == 0, lib.b2_last_error()
    assert (c.arch, c.num_layers, c.hidden, c.vocab, c.norm_groups) == (capi.ARCH_KEDASUN, 3, 12, 31, 3)
    assert abs(c.embed_scale - 3.0) < 1e-6 and abs(c.rms_eps - 1e-5) < 1e-11
    s0, s1, s2 = specs[0], specs[1], specs[2]
    assert (s0.mixer, s0.heads, s0.kv_heads, s0.dim, s0.vdim, s0.rot_dims, s0.v_mix, s0.conv_taps, s0.window) == (capi.MIXER_ATTENTION, 4, 2, 6, 5, 4, 1, 0, 0)
    assert (s0.ff, s0.ff_dim) == (capi.FF_CLAMPED_GATED, 14) and abs(s0.ff_limit - 1.5) < 1e-6 and abs(s0.rot_base - 50.0) < 1e-6
    assert (s1.mixer, s1.conv_taps, s1.window, s1.keep_first, s1.rot_dims, s1.ff) == (capi.MIXER_CONV_ATTENTION, 3, 5, 2, 0, capi.FF_NONE)
    assert s2.v_mix == 0 and abs(s1.scale - 0.3) < 1e-6
    for i, layer in enumerate(cfg["layers"]):   # the Python mirror fills the same bytes, and reads them back
        sp = capi.b2_layer_spec()
        eng._fill_layer_spec(sp, layer)
        assert bytes(sp) == bytes(specs[i])
        back = eng._layer_dict(sp)
        assert back["type"] == layer["type"] and back["mixer"].get("mask") == layer["mixer"].get("mask")
    plain = small_cfg()     # no "kv_heads": as many as query heads; no "mask": no window; no "rot": nothing rotated
    del plain["layers"][0]["mixer"]["kv_heads"], plain["layers"][0]["mixer"]["rot"], plain["layers"][1]["mixer"]["mask"]
    (tmp_path / "config.json").write_text(json.dumps(plain))
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 8) == 0, lib.b2_last_error()
    assert (specs[0].kv_heads, specs[0].rot_dims, specs[1].window, specs[1].keep_first) == (4, 0, 0, 0)
    sp = capi.b2_layer_spec()
    eng._fill_layer_spec(sp, plain["layers"][0])
    assert bytes(sp) == bytes(specs[0])
    bad = small_cfg()
    bad["layers"][1]["mlp"] = {"kind": "moe"}
    (tmp_path / "config.json").write_text(json.dumps(bad))
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 8) != 0 and b"moe" in lib.b2_last_error()
    bad = small_cfg()
    bad["layers"][0]["type"] = "latent_attention"
    (tmp_path / "config.json").write_text(json.dumps(bad))
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 8) != 0


def test_checkpoint_names_match_the_restatement(pkg):
    from importlib import import_module
    weights = import_module("aws-k8s-ansible-provisioner_b200.weights")
    cfg = small_cfg()
    w = O.random_weights(cfg, seed=1)
    shapes = weights.kedasun_tensor_shapes(cfg)
    assert set(shapes) == set(w)
    assert all(tuple(w[k].shape) == tuple(v) for k, v in shapes.items())
    assert "l1.norm2" not in w and "l1.mix.talk" in w and "l0.mix.talk" not in w


def test_grouped_norm_normalises_every_piece():
    x = torch.tensor([[3.0, 4.0, 0.0, 0.5, 100.0, -100.0]], dtype=torch.float64)
    y = O.grouped_rms_norm(x, torch.ones(6, dtype=torch.float64), 3, 0.0)
    assert torch.allclose((y.reshape(3, 2) ** 2).mean(-1), torch.ones(3, dtype=torch.float64))
    one = O.grouped_rms_norm(x, torch.ones(6, dtype=torch.float64), 1, 0.0)
    assert abs(float((one ** 2).mean()) - 1.0) < 1e-12 and abs(float(one[0, 0])) < 0.1   # one statistic: the large pair dominates


def test_rotation_is_pairwise_and_position_zero_is_identity():
    v = torch.arange(1.0, 9.0, dtype=torch.float64).reshape(1, 1, 8).repeat(3, 1, 1)
    out = O.rotate_pairs(v, torch.tensor([0, 1, 5]), 100.0, 4)
    assert torch.equal(out[0], v[0]) and torch.equal(out[:, :, 4:], v[:, :, 4:])
    a = 5 * 100.0 ** (-2.0 / 4)   # pair 1 at position 5
    assert abs(float(out[2, 0, 2]) - (3 * math.cos(a) - 4 * math.sin(a))) < 1e-12
    assert abs(float(out[2, 0, 3]) - (4 * math.cos(a) + 3 * math.sin(a))) < 1e-12


def test_convolution_is_causal_and_carries_its_tail():
    u = torch.arange(1.0, 11.0, dtype=torch.float64).reshape(5, 2)
    taps = torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]], dtype=torch.float64)   # channel 0: identity; channel 1: two steps back
    y = O.causal_short_conv(u, taps)
    assert torch.equal(y[:, 0], u[:, 0]) and y[:2, 1].tolist() == [0.0, 0.0] and torch.equal(y[2:, 1], u[:3, 1])
    both = torch.cat([O.causal_short_conv(u[:3], taps), O.causal_short_conv(u[3:], taps, before=u[1:3])])
    assert torch.equal(both, y)


def test_window_keeps_the_first_tokens_and_slopes_fall_with_distance():
    pos = torch.arange(12)
    vis = O.visible(pos, pos, 4, 2)
    assert vis[11].tolist() == [True, True] + [False] * 6 + [True] * 4
    assert vis[3].tolist() == [True] * 4 + [False] * 8 and O.visible(pos, pos, None, 0)[11].all()
    s = O.head_slopes(4, torch.float64)
    assert s.tolist() == [0.25, 0.0625, 0.015625, 0.00390625]
    q, k = torch.zeros(12, 1, 2, dtype=torch.float64), torch.zeros(12, 1, 2, dtype=torch.float64)
    v = torch.eye(12, dtype=torch.float64).reshape(12, 1, 12)
    w = O.attend(q, k, v, pos, pos, 1.0, slopes=torch.tensor([math.log(2.0)], dtype=torch.float64))[11, 0]   # the weights themselves
    assert abs(float(w[10] / w[11]) - 0.5) < 1e-12 and abs(float(w.sum()) - 1.0) < 1e-12


def test_mixed_weights_act_on_the_heads_own_values():
    torch.manual_seed(0)
    q, k, v = torch.randn(5, 4, 3, dtype=torch.float64), torch.randn(5, 2, 3, dtype=torch.float64), torch.randn(5, 2, 2, dtype=torch.float64)
    pos = torch.arange(5)
    plain = O.attend(q, k, v, pos, pos, 0.7)
    assert torch.allclose(O.attend(q, k, v, pos, pos, 0.7, talk=torch.eye(4, dtype=torch.float64)), plain)
    swap = torch.eye(4, dtype=torch.float64)[[1, 0, 2, 3]]     # heads 0 and 1 share key/value head 0: swapping their weights swaps their outputs
    sw = O.attend(q, k, v, pos, pos, 0.7, talk=swap)
    assert torch.allclose(sw[:, 0], plain[:, 1]) and torch.allclose(sw[:, 1], plain[:, 0]) and torch.allclose(sw[:, 2:], plain[:, 2:])
    cross = torch.eye(4, dtype=torch.float64)[[2, 1, 0, 3]]    # head 0 takes head 2's weights but keeps its own values
    kk, vv = k.repeat_interleave(2, 1), v.repeat_interleave(2, 1)
    s = torch.einsum("iad,jad->aij", q, kk) * 0.7
    wts = O.softmax_weights(s, O.visible(pos, pos, None, 0))
    assert torch.allclose(O.attend(q, k, v, pos, pos, 0.7, talk=cross)[:, 0], torch.einsum("ij,jd->id", wts[2], vv[:, 0]))


def test_feed_forward_clamps_before_the_gate():
    w = {"m.gate": torch.tensor([[1.0], [1.0]], dtype=torch.float64), "m.up": torch.tensor([[1.0], [-1.0]], dtype=torch.float64),
         "m.down": torch.eye(2, dtype=torch.float64)}
    y = O.clamped_gated_ff(torch.tensor([[10.0]], dtype=torch.float64), w, "m.", 2.0)
    g = 2.0 / (1.0 + math.exp(-1.702 * 2.0))
    assert torch.allclose(y, torch.tensor([[g * 3.0, g * -1.0]], dtype=torch.float64))
    y = O.clamped_gated_ff(torch.tensor([[-10.0]], dtype=torch.float64), w, "m.", 2.0)   # the gate is clamped from above only
    g = -10.0 / (1.0 + math.exp(17.02))
    assert torch.allclose(y, torch.tensor([[g * -1.0, g * 3.0]], dtype=torch.float64))


def test_restatement_stepwise_equals_whole():
    cfg = small_cfg()
    w = O.random_weights(cfg, seed=3)
    toks = torch.randint(0, cfg["vocab"], (23,), generator=torch.Generator().manual_seed(4)).tolist()
    whole, streams = O.forward(cfg, w, toks)
    o = O.Stepper(cfg, w)
    parts = [o.feed(toks[:7])[0], o.feed(toks[7:9])[0]] + [o.feed([t])[0] for t in toks[9:]]
    assert torch.allclose(torch.cat(parts), whole, rtol=1e-10, atol=1e-12)
    assert len(streams) == len(cfg["layers"]) + 1
    # the value blend reads the first mixing layer's values: changing layer 0's value weights moves layer 1 even with its output cut
    w2 = dict(w)
    w2["l1.mix.vmix"] = torch.tensor(0.0)
    assert not torch.allclose(O.forward(cfg, w2, toks)[0], whole)
