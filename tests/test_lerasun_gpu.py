"""The Lerasun family through the engine (GPU) against the plain restatement in oracle/lerasun_oracle.py.

Every test builds its own small configuration and random weights.  The engine runs in fp32 (tight bars: a lost key, a
window one token off, a stale page or a missing sink shows far above fp32 rounding) and in bf16 (loose bars).
What is covered: every layer's residual stream; whole prompts against token-by-token decoding; prompt portions down to two
tokens; unequal requests in one batch against each alone; pages and sequence slots that are freed and used again; keys far
back and at page borders with sharpened attention; the first tokens of a sequence; a long run of decode steps; sizes that
differ per layer, group selection that actually drops groups, layers without a feed-forward, layers that read another
layer's cache; greedy generation through the engine's own prefill / decode entry points and through b2serve's scheduler.
"""
import http.client
import json
import os
import subprocess
import time

import numpy as np
import pytest
import torch

from _util import pkg
from oracle.lerasun_oracle import Oracle, random_weights

pytestmark = pytest.mark.gpu


def mixer(heads, dim, rot, vdim, rank, scale, base=10000.0, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": {"base": base, "dims": rot}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def moe(ff, experts, top, groups, keep):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}}


def layer(m, mlp):
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def cfg_a():
    """Odd sizes, none a multiple of a tile; groups that are dropped; a layer with no feed-forward; two cache readers."""
    return {"architecture": "Lerasun", "vocab": 203, "width": 88, "logit_scale": 0.5, "norm": {"eps": 1e-5}, "layers": [
        layer(mixer(3, 12, 6, 20, 40, 0.3), moe(36, 6, 3, 3, 2)),
        layer(mixer(3, 12, 6, 20, 40, 0.3, kv_from=0), moe(36, 6, 3, 3, 2)),
        layer(mixer(5, 8, 10, 6, 24, 0.21, base=500.0), None),
        layer(mixer(2, 20, 10, 14, 24, 0.4, base=500.0, kv_from=2), moe(20, 8, 2, 4, 1)),
    ]}


def cfg_b():
    """One group, every expert used (top == experts), one head, latent wider than 32 lanes x 1."""
    return {"architecture": "Lerasun", "vocab": 97, "width": 64, "logit_scale": 1.0, "norm": {"eps": 1e-6}, "layers": [
        layer(mixer(1, 16, 4, 16, 72, 0.25), moe(24, 2, 2, 1, 1)),
        layer(mixer(4, 4, 2, 8, 16, 0.5, base=100.0), moe(8, 4, 1, 2, 2)),
    ]}


def cfg_c():
    """Sizes the tensor-core forms take: inner dimensions in multiples of 64, more than 64 tokens per call, logit scale 1."""
    m = mixer(4, 32, 16, 32, 128, 0.15)
    return {"architecture": "Lerasun", "vocab": 300, "width": 128, "logit_scale": 1.0, "norm": {"eps": 1e-6}, "layers": [
        layer(m, moe(64, 4, 2, 2, 1)), layer(dict(m, kv_from=0), moe(64, 4, 2, 2, 1)), layer(mixer(2, 64, 32, 64, 192, 0.1), None)]}


def sharpen(w, cfg, factor=6.0):
    """Scaled queries make every softmax peak on a few keys, wherever they are: a key that is lost shows."""
    for i, _ in enumerate(cfg["layers"]):
        w[f"l{i}.mix.q"] = (w[f"l{i}.mix.q"] * factor).to(torch.bfloat16).float()
    return w


def engine(cfg, w, f32=True, **rt):
    P = pkg()
    rt = {"max_model_len": 1024, "num_blocks": 80, "max_seqs": 4, "max_batch_tokens": 1024, **rt}
    e = P.Engine(P.EngineConfig.lerasun(cfg, compute_f32=f32, **rt))
    e.load_state_dict({k: v.to(torch.bfloat16) for k, v in w.items()})
    return e


def tokens(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def err(got, ref):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-9))


F32_BAR, BF16_BAR = 2e-5, 6e-2


def rows_over(got, ref, bar):
    """Positions whose logits differ by more than `bar`.  In bf16 a router score that is a near tie in exact arithmetic may
    fall the other way for a single token, which changes that token's experts and nothing else: the bf16 comparisons of
    long prompts allow one position in a hundred for that; every systematic fault moves far more."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    return int((np.abs(got - ref).max(1) / max(np.abs(ref).max(), 1e-9) > bar).sum())


@pytest.mark.parametrize("make", [cfg_a, cfg_b])
def test_every_layer_fp32(make):
    cfg = make()
    w = random_weights(cfg, seed=1)
    toks = tokens(cfg, 37, 2)
    ref_logits, ref_layers = Oracle(cfg, w).forward(toks, capture_layers=True)
    with engine(cfg, w) as e:
        e.set_debug(hidden=True)
        sid = e.seq_create(64)
        logits, _ = e.prefill_logits([sid], [toks], list(range(len(toks))))
        for l in range(len(cfg["layers"])):
            assert err(e.get_hidden_f32(l, len(toks)), ref_layers[l].numpy()) < F32_BAR, "residual stream after layer %d" % l
        assert err(logits, ref_logits.numpy()) < F32_BAR


@pytest.mark.parametrize("make", [cfg_a, cfg_b])
def test_bf16_close_to_oracle(make):
    cfg = make()
    w = random_weights(cfg, seed=3)
    toks = tokens(cfg, 50, 4)
    ref = Oracle(cfg, w).forward(toks).numpy()
    with engine(cfg, w, f32=False) as e:
        sid = e.seq_create(64)
        logits, _ = e.prefill_logits([sid], [toks[:41]], list(range(41)))
        assert err(logits, ref[:41]) < BF16_BAR
        for p in range(41, 50):
            e.decode_step([sid], in_tokens=[toks[p]], want_output=False)
            assert err(e.get_logits(1)[0], ref[p]) < BF16_BAR


def test_bf16_prompt_sized_and_decode_sized_kernels_agree():
    """bf16: a 330-token prompt (tcgen05 projections, 64-row MMA tiles, 64-key attention tiles with a ragged last tile) against the
    oracle, then the same positions decoded one by one (weight-streaming products, key splits + merge) against both."""
    cfg = cfg_c()
    w = random_weights(cfg, seed=23)
    toks = tokens(cfg, 330, 24)
    ref = Oracle(cfg, w).forward(toks).numpy()
    with engine(cfg, w, f32=False) as e:
        a = e.seq_create(400)
        lw, _ = e.prefill_logits([a], [toks], list(range(330)))
        assert rows_over(lw, ref, BF16_BAR) <= 3
        b = e.seq_create(400)
        e.prefill_logits([b], [toks[:70]], [])
        e.prefill_logits([b], [toks[70:300]], [])
        dec = []
        for p in range(300, 330):
            e.decode_step([b], in_tokens=[toks[p]], want_output=False)
            dec.append(e.get_logits(1)[0])
        assert rows_over(np.stack(dec), ref[300:], BF16_BAR) <= 1 and rows_over(np.stack(dec), lw[300:], BF16_BAR) <= 1


def test_bf16_expert_products_of_a_long_step():
    """bf16: a step with more than 2048 (token, choice) pairs runs every expert's two products as dense tcgen05 projections over
    rows gathered into expert order; shorter steps run them as ragged groups.  Two unequal prompts in one long step against the
    oracle and against the same prompts fed in short portions.  One expert's correction keeps it from ever being chosen, so an
    empty slot range is among the experts."""
    m = mixer(2, 32, 16, 32, 64, 0.2)
    cfg = {"architecture": "Lerasun", "vocab": 211, "width": 128, "logit_scale": 0.5, "norm": {"eps": 1e-6}, "layers": [
        layer(m, moe(128, 5, 2, 1, 1)), layer(dict(m, kv_from=0), moe(192, 6, 3, 3, 2))]}
    w = random_weights(cfg, seed=41)
    w["l0.mlp.correction"][3] = -50.0
    prompts = [tokens(cfg, 640, 42), tokens(cfg, 470, 43)]
    refs = [Oracle(cfg, w).forward(p).numpy() for p in prompts]
    with engine(cfg, w, f32=False, max_batch_tokens=1280, num_blocks=200) as e:
        sids = [e.seq_create(700), e.seq_create(700)]
        rows = list(range(600, 640)) + list(range(640 + 430, 640 + 470))
        long_step, _ = e.prefill_logits(sids, prompts, rows)
        ref = np.concatenate([refs[0][600:], refs[1][430:]])
        assert rows_over(long_step, ref, BF16_BAR) <= 1
        t = [e.seq_create(700), e.seq_create(700)]
        for lo in range(0, 400, 200):
            e.prefill_logits(t, [p[lo:lo + 200] for p in prompts], [])
        short = [e.prefill_logits([t[i]], [prompts[i][400:]], list(range(len(prompts[i]) - 440, len(prompts[i]) - 400)))[0] for i in range(2)]
        assert rows_over(np.concatenate(short), long_step, BF16_BAR) <= 1


@pytest.mark.parametrize("experts,groups,keep,top", [(1, 1, 1, 1), (3, 1, 1, 2), (5, 5, 3, 2), (7, 1, 1, 7), (9, 3, 2, 4), (15, 5, 2, 1), (34, 2, 1, 17)])
def test_router_of_any_expert_count(experts, groups, keep, top):
    """Expert counts that are odd, prime, one, or more than a warp's lanes, with a width the router reads four numbers at a time:
    fp32 engine against the oracle on a prompt and a few decoded tokens (a wrong choice or weight moves the logits far above fp32 rounding)."""
    cfg = {"architecture": "Lerasun", "vocab": 61, "width": 72, "logit_scale": 1.0, "norm": {"eps": 1e-6}, "layers": [
        layer(mixer(2, 8, 4, 8, 16, 0.3), moe(12, experts, top, groups, keep)), layer(mixer(2, 8, 4, 8, 16, 0.3, kv_from=0), moe(20, experts, top, groups, keep))]}
    w = random_weights(cfg, seed=50 + experts)
    toks = tokens(cfg, 45, 51)
    ref = Oracle(cfg, w).forward(toks).numpy()
    with engine(cfg, w) as e:
        sid = e.seq_create(64)
        lg, _ = e.prefill_logits([sid], [toks[:40]], list(range(40)))
        assert err(lg, ref[:40]) < F32_BAR
        for p in range(40, 45):
            e.decode_step([sid], in_tokens=[toks[p]], want_output=False)
            assert err(e.get_logits(1)[0], ref[p]) < F32_BAR


@pytest.mark.parametrize("nseq", [3, 12, 27, 50])
def test_bf16_decode_batches_of_many_sizes(nseq):
    """bf16 decode steps whose batch fills one, two, four and eight 8-row token tiles of the weight-streaming products (and
    leaves the last tile ragged), sequences of unequal length: every sequence's logits against the oracle's for that sequence
    alone, and against the same sequence decoded in a batch of one."""
    cfg = cfg_c()
    w = random_weights(cfg, seed=31)
    prompts = [tokens(cfg, 3 + (7 * i) % 41, 100 + i) for i in range(nseq)]
    refs = [Oracle(cfg, w).forward(p).numpy()[-1] for p in prompts]   # (an oracle holds one sequence)
    with engine(cfg, w, f32=False, max_seqs=nseq, num_blocks=4 * nseq + 8, max_model_len=64, max_batch_tokens=2048) as e:
        sids = [e.seq_create(64) for _ in prompts]
        e.prefill_logits(sids, [p[:-1] for p in prompts], [])
        e.decode_step(sids, in_tokens=[p[-1] for p in prompts], want_output=False)
        lg = e.get_logits(nseq)
        assert rows_over(lg, np.stack(refs), BF16_BAR) <= max(1, nseq // 25)
    with engine(cfg, w, f32=False, max_seqs=1, num_blocks=12, max_model_len=64, max_batch_tokens=64) as e:
        k = nseq - 1
        alone = e.seq_create(64)
        e.prefill_logits([alone], [prompts[k][:-1]], [])
        e.decode_step([alone], in_tokens=[prompts[k][-1]], want_output=False)
        assert rows_over(e.get_logits(1), lg[k:k + 1], BF16_BAR) == 0


def test_prefill_against_token_by_token_decoding():
    cfg = cfg_a()
    w = sharpen(random_weights(cfg, seed=5), cfg)
    toks = tokens(cfg, 70, 6)
    ref = Oracle(cfg, w).forward(toks).numpy()
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


@pytest.mark.parametrize("cuts", [[2, 2, 2, 64, 3, 17, 2, 31], [16, 16, 32, 1, 1, 57], [63, 2, 58]])
def test_portions_of_a_prompt(cuts):
    cfg = cfg_a()
    w = sharpen(random_weights(cfg, seed=7), cfg)
    n = sum(cuts)
    toks = tokens(cfg, n, 8)
    ref = Oracle(cfg, w).forward(toks).numpy()
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
    refs = [Oracle(cfg, w).forward(p).numpy() for p in prompts]
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
        # a pure decode batch of unequal lengths (the captured step), against the same references
        live = [0, 2]
        e.decode_step([sids[r] for r in live], in_tokens=[prompts[r][done[r]] for r in live], want_output=False)
        lg = e.get_logits(2)
        for k, r in enumerate(live):
            assert err(lg[k], refs[r][done[r]]) < F32_BAR


def test_pages_and_slots_are_used_again():
    cfg = cfg_b()
    w = sharpen(random_weights(cfg, seed=11), cfg)
    with engine(cfg, w, num_blocks=9, max_seqs=2, max_model_len=128, max_batch_tokens=128) as e:   # 8 usable pages = 128 tokens
        for rnd in range(5):
            n = [100, 28][rnd % 2] if rnd < 4 else 120
            toks = tokens(cfg, n, 30 + rnd)
            ref = Oracle(cfg, w).forward(toks).numpy()
            sid = e.seq_create(16)
            other = e.seq_create(8) if rnd % 2 else None   # a second live request takes pages in between
            at = 0
            for c in [16, n - 16 - 4, 1, 1, 1, 1]:
                e.seq_reserve(sid, at + c)
                lg, _ = e.prefill_logits([sid], [toks[at:at + c]], list(range(c)))
                assert err(lg, ref[at:at + c]) < F32_BAR, "round %d at %d" % (rnd, at)
                at += c
            e.seq_free(sid)
            if other is not None:
                e.seq_free(other)
        assert e.info()["free_blocks"] == 8


def test_far_keys_and_page_borders():
    """One token id occurs once, far back; every layer's queries are scaled up, so late positions lean on single keys."""
    cfg = cfg_b()
    w = sharpen(random_weights(cfg, seed=13), cfg, factor=10.0)
    n = 600
    toks = tokens(cfg, n, 14)
    ref = Oracle(cfg, w).forward(toks).numpy()
    want = [0, 1, 2, 15, 16, 17, 31, 32, 33, 255, 256, 257, 511, 512, 513, 598, 599]
    with engine(cfg, w, num_blocks=100) as e:
        sid = e.seq_create(n + 40)
        lg, _ = e.prefill_logits([sid], [toks], want)
        assert err(lg, ref[want]) < F32_BAR
        # the same positions reached by decoding over page borders (positions 560..599 decoded one by one)
        sid2 = e.seq_create(n + 40)
        e.prefill_logits([sid2], [toks[:560]], [])
        for p in range(560, n):
            e.decode_step([sid2], in_tokens=[toks[p]], want_output=False)
            if p in (575, 576, 577, 591, 592, 593, 599):
                assert err(e.get_logits(1)[0], ref[p]) < F32_BAR, "decoded position %d" % p


def test_sink_counts_once_and_has_no_value():
    cfg = cfg_b()
    w = random_weights(cfg, seed=15)
    toks = tokens(cfg, 24, 16)
    for sink in (-30.0, 0.0, 4.0, 30.0):
        for i in range(len(cfg["layers"])):
            w[f"l{i}.mix.sink"] = torch.full_like(w[f"l{i}.mix.sink"], sink)
        ref = Oracle(cfg, w).forward(toks).numpy()
        with engine(cfg, w) as e:
            sid = e.seq_create(32)
            lg, _ = e.prefill_logits([sid], [toks], list(range(24)))
            assert err(lg, ref) < F32_BAR, "sink %g" % sink
    # a sink that swallows the softmax leaves the feed-forward branch alone: the mixer adds (almost) nothing
    w2 = {k: v.clone() for k, v in w.items()}
    for i in range(len(cfg["layers"])):
        w2[f"l{i}.mix.o"] = torch.zeros_like(w2[f"l{i}.mix.o"])
    ref_no_mixer = Oracle(cfg, w2).forward(toks).numpy()
    assert err(lg, ref_no_mixer) < 1e-6


def test_long_decoding():
    cfg = cfg_a()
    w = sharpen(random_weights(cfg, seed=17), cfg)
    n = 230
    toks = tokens(cfg, n, 18)
    ref = Oracle(cfg, w).forward(toks).numpy()
    with engine(cfg, w) as e:
        sid = e.seq_create(n)
        e.prefill_logits([sid], [toks[:20]], [])
        worst = 0.0
        for p in range(20, n):
            e.decode_step([sid], in_tokens=[toks[p]], want_output=False)
            worst = max(worst, err(e.get_logits(1)[0], ref[p]))
        assert worst < F32_BAR


def test_greedy_generation_through_the_engine():
    cfg = cfg_a()
    w = random_weights(cfg, seed=19)
    prompts = [tokens(cfg, 33, 40), tokens(cfg, 9, 41)]
    refs = [Oracle(cfg, w).greedy(p, 12) for p in prompts]
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
    steps over the running requests) generates what the oracle generates."""
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
    proc = subprocess.Popen([exe, str(tmp_path), "--served-model-name", "lerasun-test", "--port", "0", "--host", "127.0.0.1", "--max-model-len", "256",
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
        c.request("POST", "/v1/completions", body=json.dumps({"model": "lerasun-test", "prompt": prompt, "max_tokens": 10, "temperature": 0,
                                                              "ignore_eos": True}), headers={"Content-Type": "application/json"})
        r = c.getresponse()
        body = json.loads(r.read().decode())
        assert r.status == 200, body
        ref = Oracle(cfg, w).greedy(prompt, 10)
        import re
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
