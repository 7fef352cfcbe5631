"""Host-side checks for the Lerasun family: the registry reads a model directory's config.json into the C structs, and the
plain restatement the GPU tests lean on is itself checked mechanism by mechanism on hand-made cases (no GPU)."""
import ctypes as C
import json
import math

import pytest
import torch

from oracle import lerasun_oracle as O


def small_cfg():
    m = {"heads": 2, "dim": 6, "rot_dim": 4, "vdim": 5, "kv_rank": 10, "scale": 0.4, "rot": {"base": 50.0, "dims": 4}}
    mlp = {"kind": "moe", "expert": {"ff": 7}, "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}}
    return {"architecture": "Lerasun", "vocab": 31, "width": 12, "logit_scale": 0.7, "norm": {"eps": 1e-5}, "layers": [
        {"type": "latent_attention", "mixer": dict(m), "mlp": mlp},
        {"type": "latent_attention", "mixer": dict(m, kv_from=0), "mlp": None}]}


def test_registry_reads_a_layer_list(pkg, lib, tmp_path):
    cfg = small_cfg()
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    from importlib import import_module
    capi = import_module("aws-k8s-ansible-provisioner_b200.capi")
    c = capi.b2_config()
    specs = (capi.b2_layer_spec * 8)()
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 8) == 0, lib.b2_last_error()
    assert (c.arch, c.num_layers, c.hidden, c.vocab) == (capi.ARCH_LERASUN, 2, 12, 31)
    assert abs(c.logit_scale - 0.7) < 1e-6 and abs(c.rms_eps - 1e-5) < 1e-11
    s0, s1 = specs[0], specs[1]
    assert (s0.heads, s0.dim, s0.rot_dim, s0.vdim, s0.kv_rank, s0.kv_from, s0.rot_dims) == (2, 6, 4, 5, 10, -1, 4)
    assert (s0.ff, s0.ff_dim, s0.experts, s0.top, s0.groups, s0.groups_keep) == (capi.FF_ROUTED_EXPERTS, 7, 6, 2, 3, 2)
    assert s1.kv_from == 0 and s1.ff == capi.FF_NONE and abs(s1.rot_base - 50.0) < 1e-6 and abs(s1.scale - 0.4) < 1e-6
    # too little room, an unknown architecture and an unknown mixer are refused with a message
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 1) != 0
    (tmp_path / "config.json").write_text(json.dumps(dict(cfg, architecture="Other")))
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 8) != 0 and b"Other" in lib.b2_last_error()
    bad = small_cfg()
    bad["layers"][0]["type"] = "something_else"
    (tmp_path / "config.json").write_text(json.dumps(bad))
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 8) != 0


def test_registry_still_reads_hf_configs(lib, tmp_path):
    from importlib import import_module
    capi = import_module("aws-k8s-ansible-provisioner_b200.capi")
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "phi3", "num_hidden_layers": 3, "hidden_size": 512, "num_attention_heads": 4,
                                                      "num_key_value_heads": 4, "intermediate_size": 1024, "vocab_size": 1000,
                                                      "partial_rotary_factor": 0.75, "sliding_window": 77, "tie_word_embeddings": False}))
    c = capi.b2_config()
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), None, 0) == 0
    assert (c.arch, c.num_layers, c.head_dim, c.rotary_dim, c.sliding_window, c.tie_embeddings) == (capi.ARCH_PHI3, 3, 128, 96, 77, 0)


def test_python_layer_specs_match_the_registry(pkg, lib, tmp_path):
    from importlib import import_module
    capi = import_module("aws-k8s-ansible-provisioner_b200.capi")
    eng = import_module("aws-k8s-ansible-provisioner_b200.engine")
    cfg = small_cfg()
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    c = capi.b2_config()
    specs = (capi.b2_layer_spec * 8)()
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 8) == 0
    for i, layer in enumerate(cfg["layers"]):
        sp = capi.b2_layer_spec()
        eng._fill_layer_spec(sp, layer)
        assert bytes(sp) == bytes(specs[i])
        assert eng._layer_dict(sp)["mixer"].get("kv_from") == layer["mixer"].get("kv_from")


def test_rotation_is_pairwise_and_position_zero_is_identity():
    v = torch.arange(1.0, 9.0, dtype=torch.float64).reshape(1, 8).repeat(3, 1)
    out = O.rotate_pairs(v, torch.tensor([0, 1, 5]), 100.0, 4)
    assert torch.equal(out[0], v[0])
    assert torch.equal(out[:, 4:], v[:, 4:])            # beyond the rotated dims nothing moves
    a = 5 * 100.0 ** (-2.0 / 4)                          # pair 1 at position 5
    assert abs(out[2, 2] - (3 * math.cos(a) - 4 * math.sin(a))) < 1e-12 and abs(out[2, 3] - (4 * math.cos(a) + 3 * math.sin(a))) < 1e-12
    assert abs(out[1, 0] - (math.cos(1.0) - 2 * math.sin(1.0))) < 1e-12


def test_router_groups_offsets_and_weights():
    r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}
    W = 4
    x = torch.zeros(1, W, dtype=torch.float64)
    x[0, 0] = 1.0
    router = torch.zeros(6, W, dtype=torch.float64)
    router[:, 0] = torch.tensor([2.0, -1.0, 0.5, 0.4, 3.0, -9.0])      # sigmoids .88 .27 .62 .60 .95 .0001
    corr = torch.tensor([0.0, 0.0, 0.0, 0.0, -0.9, 0.0], dtype=torch.float64)
    w = {"p.router": router, "p.correction": corr}
    idx, wt = O.route(x, w, "p.", r)
    # group scores from CHOICE scores (with the offset): g0 = .88 + .27, g1 = .62 + .60, g2 = .05 + .0001 -> g2 is out although
    # expert 4 has the best plain score; chosen: experts 0 and 2; weights from the plain scores
    assert sorted(idx[0].tolist()) == [0, 2]
    s0, s2 = torch.sigmoid(torch.tensor(2.0, dtype=torch.float64)), torch.sigmoid(torch.tensor(0.5, dtype=torch.float64))
    got = dict(zip(idx[0].tolist(), wt[0].tolist()))
    assert abs(got[0] - float(s0 / (s0 + s2))) < 1e-12 and abs(sum(wt[0].tolist()) - 1.0) < 1e-12
    # negative choice scores still beat a dropped group's experts
    corr2 = torch.tensor([-5.0, -5.0, -5.0, -5.0, 0.0, 0.0], dtype=torch.float64)
    idx2, _ = O.route(x, {"p.router": router, "p.correction": corr2}, "p.", {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}})
    assert sorted(idx2[0].tolist()) == [4, 5]


def test_sink_takes_weight_without_a_value():
    cfg = small_cfg()
    w = O.random_weights(cfg, seed=2)
    m = cfg["layers"][0]["mixer"]
    x = torch.randn(5, cfg["width"], dtype=torch.float64)
    pos = torch.arange(5)
    w64 = {k: v.double() for k, v in w.items()}
    c, kr = O.latent_and_rotated_key(x, pos, w64, "l0.mix.", m, 1e-5)
    w64["l0.mix.sink"] = torch.full((2,), -80.0, dtype=torch.float64)
    plain = O.latent_attention(x, pos, c, kr, w64, "l0.mix.", m)
    # position 0 sees one key: without a sink its softmax weight is 1; a sink equal to that one score halves it
    w64["l0.mix.sink"] = torch.full((2,), 80.0, dtype=torch.float64)
    swallowed = O.latent_attention(x, pos, c, kr, w64, "l0.mix.", m)
    assert swallowed.abs().max() < 1e-20 * max(1.0, float(plain.abs().max())) + 1e-25
    q = (x[:1] @ w64["l0.mix.q"].T).reshape(1, 2, 10)
    for a in range(2):
        kn = c[:1] @ w64["l0.mix.uk"][a * 6:(a + 1) * 6].T
        qr = O.rotate_pairs(q[:, a, 6:], pos[:1], 50.0, 4)
        w64["l0.mix.sink"][a] = ((q[0, a, :6] @ kn[0]) + (qr[0] @ kr[0])) * m["scale"]
    half = O.latent_attention(x[:1], pos[:1], c[:1], kr[:1], w64, "l0.mix.", m)
    assert torch.allclose(half, 0.5 * plain[:1], rtol=1e-10, atol=1e-14)


def test_oracle_stepwise_equals_whole():
    cfg = small_cfg()
    w = O.random_weights(cfg, seed=3)
    toks = torch.randint(0, cfg["vocab"], (23,), generator=torch.Generator().manual_seed(4)).tolist()
    whole = O.Oracle(cfg, w).forward(toks)
    o = O.Oracle(cfg, w)
    parts = [o.forward(toks[:7]), o.forward(toks[7:9])] + [o.forward([t]) for t in toks[9:]]
    assert torch.allclose(torch.cat(parts), whole, rtol=1e-10, atol=1e-12)
    assert set(O.tensor_shapes(cfg)) == set(w) and "l1.norm2" not in w and "l1.mix.dkv" not in w
