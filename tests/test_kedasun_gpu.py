"""The Kedasun family through the engine (GPU) against the plain restatement in oracle/kedasun_oracle.py.

Every test builds its own small configuration and random weights.  The engine runs in fp32 (tight bars: a lost key, a
window one token off, a stale page, a convolution that reads the wrong row shows far above fp32 rounding) and in bf16 (loose
bars).  Covered: each mechanism alone (single-layer models); every layer's residual stream; whole prompts against
token-by-token decoding; prompt portions down to two tokens; unequal requests in one batch against each alone; pages and
sequence slots freed and used again (the convolution's per-slot rows included); keys far back, at page borders and just
inside / outside the window and the kept first tokens, in prompts and in decoding; the first tokens of a sequence; a long
run of decode steps; sizes that differ per layer and values a model may make equal or one; greedy generation through the
engine's own entry points and through b2serve's scheduler.
"""
import http.client
import json
import os
import re
import subprocess
import time

import numpy as np
import pytest
import torch

from _util import pkg
from oracle.kedasun_oracle import Stepper, forward, random_weights

pytestmark = pytest.mark.gpu


def att(heads, kv, dim, vdim, scale, rot=None, base=10000.0, v_mix=True):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
    return {"type": "attention", "mixer": m}


def att2(heads, kv, dim, vdim, scale, conv, window=None, keep=0, v_mix=True):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "conv": conv, "v_mix": v_mix}
    if window is not None:
        m["mask"] = {"size": window, "keep_first": keep}
    return {"type": "attention_2", "mixer": m}


def ff(n, limit=2.0):
    return {"kind": "dense", "ff": n, "limit": limit}


def model(layers, vocab=203, width=88, groups=4, escale=5.0, eps=1e-5):
    return {"architecture": "Kedasun", "vocab": vocab, "width": width, "embedding": {"scale": escale}, "norm": {"eps": eps, "groups": groups},
            "layers": [dict(m, mlp=f) for m, f in layers]}


def cfg_a():
    """Odd sizes, none a multiple of a tile; three query heads per key/value head; the first value-mixing layer is a convolution
    layer; a layer outside the value mixing; a layer without a feed-forward; a window shorter than a page with kept tokens."""
    return model([(att2(6, 2, 10, 12, 0.9, 4, window=11, keep=3), ff(36)), (att(4, 2, 14, 12, 0.3, rot=6, base=500.0), None),
                  (att(4, 4, 12, 6, 0.25, rot=12, v_mix=False), ff(20, 0.7)), (att2(2, 2, 18, 12, 1.4, 2, window=40, keep=0), ff(52, 3.0))])


def cfg_b():
    """One head, one norm piece, no rotation at all, one tap, a window of one key (the token itself plus the kept ones), no mask."""
    return model([(att(1, 1, 16, 16, 0.25), ff(24)), (att2(1, 1, 8, 16, 1.0, 1, window=1, keep=5), ff(8)), (att2(4, 1, 4, 16, 2.0, 5), None)],
                 vocab=97, width=64, groups=1, escale=1.0, eps=1e-6)


def cfg_c():
    """Sizes the tensor-core products take: inner dimensions in multiples of 64, more than 64 tokens per call."""
    return model([(att(4, 2, 32, 32, 0.18, rot=16), ff(192)), (att2(4, 2, 32, 32, 1.2, 4, window=70, keep=9), ff(128)), (att(2, 1, 64, 64, 0.125, rot=64, v_mix=False), ff(64))],
                 vocab=300, width=128, groups=2)


def sharpen(w, cfg, factor=6.0):
    """Scaled queries make every softmax of the rotary layers peak on a few keys, wherever they are: a key that is lost shows.
    (The convolution layers normalise q and k; their sharpness is the configured score scale.)"""
    for i, L in enumerate(cfg["layers"]):
        if L["type"] == "attention":
            w[f"l{i}.mix.q"] = (w[f"l{i}.mix.q"] * factor).to(torch.bfloat16).float()
    return w


def engine(cfg, w, f32=True, **rt):
    P = pkg()
    rt = {"max_model_len": 1024, "num_blocks": 80, "max_seqs": 4, "max_batch_tokens": 1024, **rt}
    e = P.Engine(P.EngineConfig.kedasun(cfg, compute_f32=f32, **rt))
    e.load_state_dict({k: v.to(torch.bfloat16) for k, v in w.items()})
    return e


def tokens(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def ref_logits(cfg, w, toks):
    return forward(cfg, w, toks)[0].numpy()


def err(got, ref):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-9))


F32_BAR, BF16_BAR = 3e-5, 6e-2


@pytest.mark.parametrize("make", [cfg_a, cfg_b])
def test_every_layer_fp32(make):
    cfg = make()
    w = random_weights(cfg, seed=1)
    toks = tokens(cfg, 37, 2)
    logits, streams = forward(cfg, w, toks)
    with engine(cfg, w) as e:
        e.set_debug(hidden=True)
        sid = e.seq_create(64)
        got, _ = e.prefill_logits([sid], [toks], list(range(len(toks))))
        for l in range(-1, len(cfg["layers"])):
            assert err(e.get_hidden_f32(l, len(toks)), streams[l + 1].numpy()) < F32_BAR, "residual stream after layer %d" % l
        assert err(got, logits.numpy()) < F32_BAR


SINGLE = {
    "rotary, grouped queries": [(att(6, 3, 10, 7, 0.5, rot=4, base=77.0), None)],
    "every dim rotated, one kv head": [(att(4, 1, 8, 8, 0.35, rot=8), None)],
    "nothing rotated": [(att(2, 2, 9, 5, 0.4), None)],
    "feed-forward with a tight clamp": [(att(1, 1, 8, 8, 0.3, rot=2), ff(33, 0.2))],
    "convolution, window, kept tokens, mixing": [(att2(4, 2, 8, 6, 1.5, 4, window=9, keep=2), None)],
    "convolution, every key visible": [(att2(3, 3, 12, 4, 0.8, 3), None)],
    "window without kept tokens": [(att2(2, 1, 8, 8, 2.5, 2, window=17, keep=0), None)],
    "kept tokens beyond the window's reach": [(att2(2, 2, 8, 8, 2.5, 6, window=3, keep=40), None)],
    "one tap": [(att2(2, 2, 8, 8, 1.0, 1, window=6, keep=1), None)],
    "a value row wider than one pass over it": [(att2(12, 12, 8, 64, 1.0, 2, window=20, keep=3), None)],
}


@pytest.mark.parametrize("name", list(SINGLE))
def test_each_mechanism_alone(name):
    cfg = model(SINGLE[name], vocab=61, width=48, groups=3)
    w = random_weights(cfg, seed=70)
    if "l0.mix.talk" in w:   # weights far from the identity, negative ones among them
        w["l0.mix.talk"] = (torch.randn(w["l0.mix.talk"].shape, generator=torch.Generator().manual_seed(71))).to(torch.bfloat16).float()
    toks = tokens(cfg, 90, 72)
    ref = ref_logits(cfg, w, toks)
    with engine(cfg, w) as e:
        sid = e.seq_create(96)
        lg, _ = e.prefill_logits([sid], [toks[:75]], list(range(75)))
        assert err(lg, ref[:75]) < F32_BAR
        for p in range(75, 90):
            e.decode_step([sid], in_tokens=[toks[p]], want_output=False)
            assert err(e.get_logits(1)[0], ref[p]) < F32_BAR, "decoded position %d" % p


def test_norm_pieces_wider_than_a_warp_keeps():
    """One piece of 1088 numbers (more than the 512 a warp holds in registers) beside a model whose pieces are 36 wide."""
    for groups in (1, 16):
        cfg = model([(att(2, 1, 8, 8, 0.3, rot=4), ff(40)), (att2(2, 2, 8, 8, 1.1, 3, window=9, keep=2, v_mix=False), ff(24))], vocab=53, width=1088, groups=groups)
        w = random_weights(cfg, seed=80)
        toks = tokens(cfg, 30, 81)
        ref = ref_logits(cfg, w, toks)
        with engine(cfg, w) as e:
            sid = e.seq_create(32)
            lg, _ = e.prefill_logits([sid], [toks[:27]], list(range(27)))
            assert err(lg, ref[:27]) < F32_BAR
            for p in range(27, 30):
                e.decode_step([sid], in_tokens=[toks[p]], want_output=False)
                assert err(e.get_logits(1)[0], ref[p]) < F32_BAR


@pytest.mark.parametrize("make", [cfg_a, cfg_b])
def test_bf16_close_to_the_restatement(make):
    cfg = make()
    w = random_weights(cfg, seed=3)
    toks = tokens(cfg, 50, 4)
    ref = ref_logits(cfg, w, toks)
    with engine(cfg, w, f32=False) as e:
        sid = e.seq_create(64)
        logits, _ = e.prefill_logits([sid], [toks[:41]], list(range(41)))
        assert err(logits, ref[:41]) < BF16_BAR
        for p in range(41, 50):
            e.decode_step([sid], in_tokens=[toks[p]], want_output=False)
            assert err(e.get_logits(1)[0], ref[p]) < BF16_BAR


def test_bf16_prompt_sized_and_decode_sized_kernels_agree():
    """bf16: a 330-token prompt (tensor-core projections, 64-token attention tiles with a ragged last one) against the restatement,
    then the same positions decoded one by one (weight-streaming products, key splits) against both."""
    cfg = cfg_c()
    w = random_weights(cfg, seed=23)
    toks = tokens(cfg, 330, 24)
    ref = ref_logits(cfg, w, toks)
    with engine(cfg, w, f32=False) as e:
        a = e.seq_create(400)
        lw, _ = e.prefill_logits([a], [toks], list(range(330)))
        assert err(lw, ref) < BF16_BAR
        b = e.seq_create(400)
        e.prefill_logits([b], [toks[:70]], [])
        e.prefill_logits([b], [toks[70:300]], [])
        dec = []
        for p in range(300, 330):
            e.decode_step([b], in_tokens=[toks[p]], want_output=False)
            dec.append(e.get_logits(1)[0])
        assert err(np.stack(dec), ref[300:]) < BF16_BAR and err(np.stack(dec), lw[300:]) < BF16_BAR


def test_bf16_pairs_of_128_wide_heads():
    """bf16, rotary layers with 128-wide heads in groups of two: their caches take the page layout of the engine's GQA attention kernels
    (tensor-core prompt pass, page-balanced decode pass).  Value mixing crosses from such a layer into a convolution layer that keeps the plain
    layout.  A long prompt, portions that end inside tiles and pages, single tokens inside a mixed step, a decode batch of unequal lengths."""
    cfg = model([(att(4, 2, 128, 128, 128 ** -0.5, rot=64), ff(128)), (att2(2, 2, 32, 128, 0.25, 3, window=50, keep=4), ff(64)),
                 (att(2, 1, 128, 128, 0.1, rot=128, base=500.0, v_mix=False), None)], vocab=300, width=128, groups=2)
    w = random_weights(cfg, seed=61)
    prompts = [tokens(cfg, 330, 62), tokens(cfg, 75, 63)]
    refs = [ref_logits(cfg, w, p) for p in prompts]
    with engine(cfg, w, f32=False) as e:
        a = e.seq_create(400)
        lw, _ = e.prefill_logits([a], [prompts[0]], list(range(330)))
        assert err(lw, refs[0]) < BF16_BAR
        sids = [e.seq_create(400), e.seq_create(100)]
        done = [0, 0]
        for step in ([(0, 70), (1, 3)], [(0, 201), (1, 1)], [(0, 1), (1, 60)], [(0, 30), (1, 1)]):
            chunks, rows, base = [], [], 0
            for rq, c in step:
                chunks.append(prompts[rq][done[rq]:done[rq] + c])
                rows += list(range(base, base + c))
                base += c
            lg, _ = e.prefill_logits([sids[rq] for rq, _ in step], chunks, rows)
            base = 0
            for rq, c in step:
                assert err(lg[base:base + c], refs[rq][done[rq]:done[rq] + c]) < BF16_BAR, "request %d at %d" % (rq, done[rq])
                base += c
                done[rq] += c
        while done[1] < 75:
            e.decode_step(sids, in_tokens=[prompts[0][done[0]], prompts[1][done[1]]], want_output=False)
            lg = e.get_logits(2)
            for rq in (0, 1):
                assert err(lg[rq], refs[rq][done[rq]]) < BF16_BAR, "decoded request %d at %d" % (rq, done[rq])
                done[rq] += 1
    with engine(cfg, w) as e:     # the same model in fp32 keeps the plain layout everywhere
        a = e.seq_create(100)
        lw, _ = e.prefill_logits([a], [prompts[1]], list(range(75)))
        assert err(lw, refs[1]) < F32_BAR


@pytest.mark.parametrize("nseq", [3, 12, 27])
def test_bf16_decode_batches_of_many_sizes(nseq):
    cfg = cfg_c()
    w = random_weights(cfg, seed=31)
    prompts = [tokens(cfg, 3 + (7 * i) % 41, 100 + i) for i in range(nseq)]
    refs = [ref_logits(cfg, w, p)[-1] for p in prompts]
    with engine(cfg, w, f32=False, max_seqs=nseq, num_blocks=4 * nseq + 8, max_model_len=64, max_batch_tokens=2048) as e:
        sids = [e.seq_create(64) for _ in prompts]
        e.prefill_logits(sids, [p[:-1] for p in prompts], [])
        e.decode_step(sids, in_tokens=[p[-1] for p in prompts], want_output=False)
        assert err(e.get_logits(nseq), np.stack(refs)) < BF16_BAR


def test_prefill_against_token_by_token_decoding():
    cfg = cfg_a()
    w = sharpen(random_weights(cfg, seed=5), cfg)
    toks = tokens(cfg, 70, 6)
    ref = ref_logits(cfg, w, toks)
    with engine(cfg, w) as e:
        whole = e.seq_create(80)
        lw, _ = e.prefill_logits([whole], [toks], list(range(70)))
        assert err(lw, ref) < F32_BAR
        one = e.seq_create(80)     # the first token as a one-token prompt, everything after it as decode steps
        l0, _ = e.prefill_logits([one], [toks[:1]], [0])
        assert err(l0[0], ref[0]) < F32_BAR
        for p in range(1, 70):
            e.decode_step([one], in_tokens=[toks[p]], want_output=False)
            got = e.get_logits(1)[0]
            assert err(got, ref[p]) < F32_BAR, "decoded position %d" % p
            assert err(got, lw[p]) < F32_BAR


@pytest.mark.parametrize("cuts", [[2, 2, 2, 64, 3, 17, 2, 31], [16, 16, 32, 1, 1, 57], [63, 2, 58], [1, 1, 1, 2, 1, 3, 100]])
def test_portions_of_a_prompt(cuts):
    cfg = cfg_a()
    w = sharpen(random_weights(cfg, seed=7), cfg)
    n = sum(cuts)
    toks = tokens(cfg, n, 8)
    ref = ref_logits(cfg, w, toks)
    with engine(cfg, w) as e:
        sid = e.seq_create(n)
        at = 0
        for c in cuts:
            lg, _ = e.prefill_logits([sid], [toks[at:at + c]], list(range(c)))
            assert err(lg, ref[at:at + c]) < F32_BAR, "portion at %d of %d tokens" % (at, c)
            at += c


def test_mixed_batch_equals_each_alone():
    cfg = cfg_a()
    w = sharpen(random_weights(cfg, seed=9), cfg)
    lens = [140, 5, 60, 1]
    prompts = [tokens(cfg, n, 20 + i) for i, n in enumerate(lens)]
    refs = [ref_logits(cfg, w, p) for p in prompts]
    with engine(cfg, w) as e:
        sids = [e.seq_create(160) for _ in prompts]
        done = [0, 0, 0, 0]
        # unequal portions beside single tokens, several steps; request 3 is one token long and joins late
        plan = [[(0, 64), (1, 3)], [(0, 2), (1, 1), (2, 40)], [(0, 60), (1, 1), (2, 1), (3, 1)], [(0, 4), (2, 6)]]
        for step in plan:
            chunks, rows, base = [], [], 0
            for r, c in step:
                chunks.append(prompts[r][done[r]:done[r] + c])
                rows += list(range(base, base + c))
                base += c
            lg, _ = e.prefill_logits([sids[r] for r, _ in step], chunks, rows)
            base = 0
            for r, c in step:
                assert err(lg[base:base + c], refs[r][done[r]:done[r] + c]) < F32_BAR, "request %d at %d" % (r, done[r])
                base += c
                done[r] += c
        # pure decode batches of unequal lengths (the captured step) in two orders, against the same references
        for live in ([0, 2], [2, 0], [0]):
            e.decode_step([sids[r] for r in live], in_tokens=[prompts[r][done[r]] for r in live], want_output=False)
            lg = e.get_logits(len(live))
            for k, r in enumerate(live):
                assert err(lg[k], refs[r][done[r]]) < F32_BAR, "decode batch %r, request %d" % (live, r)
                done[r] += 1


def test_pages_and_slots_are_used_again():
    """Eight usable pages, two sequence slots: every round frees its request, the next one gets the same slot (and with it the rows
    the last request's convolutions left) and the same pages in another order."""
    cfg = cfg_b()
    w = random_weights(cfg, seed=11)
    with engine(cfg, w, num_blocks=9, max_seqs=2, max_model_len=128, max_batch_tokens=128) as e:
        for rnd in range(5):
            n = [100, 28][rnd % 2] if rnd < 4 else 120
            toks = tokens(cfg, n, 30 + rnd)
            ref = ref_logits(cfg, w, toks)
            sid = e.seq_create(16)
            other = e.seq_create(8) if rnd % 2 else None   # a second live request takes pages in between
            at = 0
            for c in [16, n - 16 - 4, 1, 1, 1, 1]:
                e.seq_reserve(sid, at + c)
                if c == 1 and at % 2:
                    e.decode_step([sid], in_tokens=[toks[at]], want_output=False)
                    lg = e.get_logits(1)
                else:
                    lg, _ = e.prefill_logits([sid], [toks[at:at + c]], list(range(c)))
                assert err(lg, ref[at:at + c]) < F32_BAR, "round %d at %d" % (rnd, at)
                at += c
            e.seq_free(sid)
            if other is not None:
                e.seq_free(other)
        assert e.info()["free_blocks"] == 8


def test_window_edges_kept_tokens_and_far_keys():
    """A sharp convolution layer (large score scale, so single keys carry the weight) with a window that ends inside a page and
    kept first tokens, under a rotary layer with scaled queries: positions around every edge, in a prompt and decoded."""
    cfg = model([(att(2, 2, 16, 8, 0.25, rot=8), ff(24)), (att2(4, 2, 8, 8, 6.0, 3, window=37, keep=5), None), (att2(2, 2, 8, 8, 6.0, 2, window=200, keep=19), ff(16))],
                vocab=97, width=64, groups=2)
    w = sharpen(random_weights(cfg, seed=13), cfg, factor=10.0)
    n = 600
    toks = tokens(cfg, n, 14)
    ref = ref_logits(cfg, w, toks)
    want = [0, 1, 2, 3, 4, 5, 6, 15, 16, 17, 18, 19, 20, 31, 32, 33, 35, 36, 37, 38, 41, 42, 43, 198, 199, 200, 201, 218, 219, 220, 255, 256, 257, 511, 512, 513, 598, 599]
    with engine(cfg, w, num_blocks=100) as e:
        sid = e.seq_create(n + 40)
        lg, _ = e.prefill_logits([sid], [toks], want)
        assert err(lg, ref[want]) < F32_BAR
        sid2 = e.seq_create(n + 40)    # the same edges crossed by decoding
        e.prefill_logits([sid2], [toks[:30]], [])
        for p in range(30, 260):
            e.decode_step([sid2], in_tokens=[toks[p]], want_output=False)
            if p in want or p % 16 in (0, 15):
                assert err(e.get_logits(1)[0], ref[p]) < F32_BAR, "decoded position %d" % p
    # the window really is part of the result: one key more or one fewer moves the logits far above the bar
    wider = json.loads(json.dumps(cfg))
    wider["layers"][1]["mixer"]["mask"]["size"] = 38
    assert err(ref_logits(wider, w, toks[:60])[40:], ref[40:60]) > 100 * F32_BAR


def test_long_decoding():
    cfg = cfg_a()
    w = sharpen(random_weights(cfg, seed=17), cfg)
    n = 230
    toks = tokens(cfg, n, 18)
    ref = ref_logits(cfg, w, toks)
    with engine(cfg, w) as e:
        sid = e.seq_create(n)
        e.prefill_logits([sid], [toks[:20]], [])
        worst = 0.0
        for p in range(20, n):
            e.decode_step([sid], in_tokens=[toks[p]], want_output=False)
            worst = max(worst, err(e.get_logits(1)[0], ref[p]))
        assert worst < F32_BAR


def test_a_sequence_cut_back_to_nothing_starts_over():
    cfg = cfg_b()
    w = random_weights(cfg, seed=41)
    toks = tokens(cfg, 40, 42)
    ref = ref_logits(cfg, w, toks)
    P = pkg()
    with engine(cfg, w) as e:
        sid = e.seq_create(64)
        e.prefill_logits([sid], [tokens(cfg, 33, 43)], [])
        with pytest.raises(P.B2Error):
            e.seq_truncate(sid, 10)     # the convolutions' rows exist for the end of the sequence only
        e.seq_truncate(sid, 0)
        lg, _ = e.prefill_logits([sid], [toks], list(range(40)))
        assert err(lg, ref) < F32_BAR


def test_blend_weight_is_needed_only_where_values_are_blended():
    cfg = cfg_a()     # layer 0 supplies the first values, layers 1 and 3 blend, layer 2 stays out
    w = random_weights(cfg, seed=45)
    toks = tokens(cfg, 20, 46)
    ref = ref_logits(cfg, w, toks)
    P = pkg()
    lean = {k: v for k, v in w.items() if k not in ("l0.mix.vmix", "l2.mix.vmix")}
    with engine(cfg, lean) as e:
        sid = e.seq_create(32)
        lg, _ = e.prefill_logits([sid], [toks], list(range(20)))
        assert err(lg, ref) < F32_BAR
    with pytest.raises(P.B2Error):
        engine(cfg, {k: v for k, v in w.items() if k != "l3.mix.vmix"})


MMA_SIZES = [(32, 32), (64, 32), (64, 64), (96, 64), (96, 96), (128, 64), (128, 128), (192, 128), (256, 128)]


def random_model(seed):
    """A random layer list: head counts, sizes (among them every pair the tensor-core prompt kernel is built for), windows, kept
    tokens, taps, rotated dims, norm pieces, layer order, value mixing and feed-forwards all drawn from the seed."""
    import random
    r = random.Random(seed)
    kv = r.choice([1, 2, 3])
    heads = kv * r.choice([1, 2, 3])
    vdim = r.choice([32, 64, 96, 128]) if seed % 2 else r.choice([5, 12, 40])
    layers = []
    for li in range(r.choice([2, 3, 4])):
        dim, vd = r.choice([(d, v) for d, v in MMA_SIZES if v == vdim] or [(r.choice([6, 20, 44]), vdim)])
        if seed % 2 == 0:
            dim = r.choice([6, 20, 44])
        mix = r.random() < 0.7
        h, g = (heads, kv) if mix else (r.choice([1, 2, 4]), 1)
        v = vd if mix else r.choice([8, 32])
        if r.random() < 0.5:
            m = att(h, g, dim, v, dim ** -0.5 * r.choice([1.0, 3.0]), rot=r.choice([0, 2, dim // 2 // 2 * 2, dim]) or None, base=r.choice([100.0, 10000.0]), v_mix=mix)
        else:
            win = r.choice([None, 1, 7, 33, 64, 100])
            m = att2(h, g, dim, v, r.choice([4.0, 12.0]) / dim, r.choice([1, 2, 3, 4]), window=win, keep=r.choice([0, 1, 9, 70]), v_mix=mix)   # unit-RMS q and k: |q.k| <= dim
        layers.append((m, ff(r.choice([24, 64, 100]), r.choice([0.5, 2.0, 7.0])) if r.random() < 0.8 else None))
    width = r.choice([64, 96, 128])
    return model(layers, vocab=r.choice([50, 131, 256]), width=width, groups=r.choice([1, 2, 4, 8]), escale=r.choice([1.0, 4.0]))


@pytest.mark.parametrize("seed", list(range(12)))
def test_random_models_and_schedules(seed):
    """fp32 and bf16 engines against the restatement on a random model: two requests, a long and a short one, fed in portions of
    uneven size in one batch (the long one past the 64-token tiles of the prompt kernels), then decoded together."""
    cfg = random_model(seed)
    w = random_weights(cfg, seed=200 + seed)
    for name in list(w):
        if name.endswith("mix.talk"):
            w[name] = (torch.eye(w[name].shape[0]) + 0.5 * torch.randn(w[name].shape, generator=torch.Generator().manual_seed(seed))).to(torch.bfloat16).float()
    prompts = [tokens(cfg, 190, 300 + seed), tokens(cfg, 23, 400 + seed)]
    refs = [ref_logits(cfg, w, p) for p in prompts]
    for f32, bar in ((True, 1e-4), (False, BF16_BAR)):   # (fp32: some of these models are sharp enough to triple fp32 rounding)
        with engine(cfg, w, f32=f32) as e:
            sids = [e.seq_create(200), e.seq_create(32)]
            done = [0, 0]
            for step in ([(0, 70), (1, 2)], [(0, 97), (1, 11)], [(0, 3), (1, 1)], [(0, 1), (1, 2)]):
                chunks, rows, base = [], [], 0
                for rq, c in step:
                    chunks.append(prompts[rq][done[rq]:done[rq] + c])
                    rows += list(range(base, base + c))
                    base += c
                lg, _ = e.prefill_logits([sids[rq] for rq, _ in step], chunks, rows)
                base = 0
                for rq, c in step:
                    assert err(lg[base:base + c], refs[rq][done[rq]:done[rq] + c]) < bar, "%s request %d at %d" % ("fp32" if f32 else "bf16", rq, done[rq])
                    base += c
                    done[rq] += c
            while done[1] < len(prompts[1]):
                e.decode_step(sids, in_tokens=[prompts[0][done[0]], prompts[1][done[1]]], want_output=False)
                lg = e.get_logits(2)
                for rq in (0, 1):
                    assert err(lg[rq], refs[rq][done[rq]]) < bar, "%s decoded request %d at %d" % ("fp32" if f32 else "bf16", rq, done[rq])
                    done[rq] += 1


def test_greedy_generation_through_the_engine():
    cfg = cfg_a()
    w = random_weights(cfg, seed=19)
    prompts = [tokens(cfg, 33, 40), tokens(cfg, 9, 41)]
    refs = [Stepper(cfg, w).greedy(p, 12) for p in prompts]
    with engine(cfg, w) as e:
        sids = [e.seq_create(64) for _ in prompts]
        out = [e.prefill(sids, prompts)]
        for _ in range(11):
            out.append(e.decode_step(sids))          # the token feedback stays on the device
        got = np.stack(out, axis=1)
        for i in range(2):
            assert got[i].tolist() == refs[i], (got[i].tolist(), refs[i])


def test_greedy_generation_through_the_server(tmp_path):
    """b2serve picks the family from config.json, loads model.safetensors, and its scheduler (chunked prefill, then decode
    steps over the running requests) generates what the restatement generates."""
    P = pkg()
    import importlib
    weights = importlib.import_module("aws-k8s-ansible-provisioner_b200.weights")
    exe = os.path.join(os.path.dirname(P.LIB_PATH), "b2serve")
    assert os.path.exists(exe), "b2serve not built"
    cfg = cfg_a()
    cfg["vocab"] = 1000         # the byte tokenizer renders ids >= 256 as <|id|>: those are read back from the reply's text
    w = random_weights(cfg, seed=21)
    weights.write_safetensors({k: v.to(torch.bfloat16) for k, v in w.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    proc = subprocess.Popen([exe, str(tmp_path), "--served-model-name", "kedasun-test", "--port", "0", "--host", "127.0.0.1", "--max-model-len", "256",
                             "--max-num-seqs", "4", "--num-gpu-blocks-override", "64", "--max-num-batched-tokens", "32", "--eos-token-id", "-1",
                             "--dtype", "float32"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        port, t0 = None, time.time()
        while time.time() - t0 < 120:
            line = proc.stdout.readline()
            if line.startswith("READY"):
                port = int(line.split()[1])
                break
            if proc.poll() is not None:
                break
        assert port is not None, "b2serve did not start: " + proc.stderr.read()
        prompt = tokens(cfg, 70, 22)   # longer than --max-num-batched-tokens: prefilled in three portions
        c = http.client.HTTPConnection("127.0.0.1", port, timeout=120)
        c.request("POST", "/v1/completions", body=json.dumps({"model": "kedasun-test", "prompt": prompt, "max_tokens": 10, "temperature": 0,
                                                              "ignore_eos": True}), headers={"Content-Type": "application/json"})
        r = c.getresponse()
        body = json.loads(r.read().decode())
        assert r.status == 200, body
        ref = Stepper(cfg, w).greedy(prompt, 10)
        got_big = [int(x) for x in re.findall(r"<\|(\d+)\|>", body["choices"][0]["text"])]
        ref_big = [t for t in ref if t >= 256]
        assert body["usage"]["completion_tokens"] == 10
        assert len(ref_big) >= 5 and got_big == ref_big, (body["choices"][0]["text"], ref)
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=10)
        except Exception:
            proc.kill()
