"""The hybrid family against the plain oracle of ``hybrid_oracle.py``.

Every test builds its own small configuration with random weights, so nothing depends on a particular checkpoint.
Sizes are chosen to be awkward on purpose: value width != key width and not a multiple of 32, fewer key heads than
value heads, rotary on only part of the rotated slice, a looped span that does not start at layer 0, a layer
without feed-forward, convolutions of 1, 2 and 4 taps.  The same tests run on the CPU (PyTorch bodies of the
operations) and, marked ``gpu``, on the sm_100a kernels in fp32 and bf16.
"""
from __future__ import annotations

import copy
import json
import os
import subprocess
import sys
import threading

import pytest
import torch

import hybrid_oracle as O
from mdi_llm_b200.models.config import HybridConfig
from mdi_llm_b200.models.hybrid import HybridLM, load_hybrid, write_safetensors
from mdi_llm_b200.ops.hybrid import BatchPlan
from mdi_llm_b200.parallel.hybrid_runner import HybridRunner
from mdi_llm_b200.parallel.scheduler import SamplingParams, starter_loop
from mdi_llm_b200.parallel.transport.inproc import LoopbackTransport

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

LATENT = {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 40},
          "mixer": {"heads": 3, "dim": 8, "rot_dim": 8, "vdim": 12, "kv_rank": 20, "q_rank": 14, "scale": 0.3,
                    "rot": {"dims": 4, "base": 100.0}}}
GLA = {"type": "gla", "mlp": None, "mixer": {"heads": 2, "dim": 8, "vdim": 20, "tau": 7.0}}
DELTA = {"type": "channel_delta", "mlp": {"kind": "dense", "ff": 56},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 10, "conv": 4}}


def cfg_dict(layers, loop=None, cap=12.0, width=24, vocab=50):
    d = {"architecture": "Badapel", "vocab": vocab, "width": width, "layers": copy.deepcopy(layers), "norm": {"eps": 1e-5}}
    if loop:
        d["loop"] = loop
    if cap:
        d["logit_softcap"] = cap
    return d


FULL = cfg_dict([GLA, LATENT, DELTA, GLA, LATENT], loop={"start": 1, "stop": 3, "times": 2})

DEVICES = [pytest.param(("cpu", torch.float32), id="cpu-f32"),
           pytest.param(("cuda", torch.float32), id="cuda-f32", marks=pytest.mark.gpu),
           pytest.param(("cuda", torch.bfloat16), id="cuda-bf16", marks=pytest.mark.gpu)]


def build(d, dev, seed=0, ranks=None):
    device, dtype = dev
    if device == "cuda":
        torch.backends.cuda.matmul.allow_tf32 = False
    model = HybridLM(HybridConfig.from_dict(d), ranks or {"l0.mix.a1": 5, "l2.mix.g1": 3}).init_random(device, dtype, seed)
    return model


def oracle_logits(d, model, tokens):
    W = {k: v.detach().cpu() for k, v in model.state_tensors().items()}
    return O.forward(d, W, list(tokens), torch.float64).float()


def tol(dev):
    return 2e-4 if dev[1] == torch.float32 else 0.25


def close(got, want, dev, what=""):
    """fp32: every logit within 2e-4.  bf16 (activations rounded to 8 bits of mantissa between operations): per row,
    the error (root mean square over the vocabulary) relative to the row's own spread is below 8 % on average and
    below 40 % at the worst row.  The models here are a few dozen channels wide, so a rounding error is averaged
    over far fewer terms than in a real layer, and single positions where a unit-normed key or a soft-max is close
    to a tie amplify it; the PyTorch bodies run in bf16 show the same figures as the kernels."""
    diff = got.float().cpu() - want
    if dev[1] == torch.float32:
        err = diff.abs().max().item()
        assert err < tol(dev), f"{what}: max abs error {err}"
        return
    rel = diff.pow(2).mean(-1).sqrt() / want.std(-1).clamp_min(1e-3)
    assert rel.mean().item() < 0.08 and rel.max().item() < 0.4, f"{what}: relative rms error mean {rel.mean()} max {rel.max()}"


def toks(n, vocab=50, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def all_rows(n):
    return [list(range(n))]


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("layer", [LATENT, GLA, DELTA], ids=["latent", "gla", "delta"])
def test_each_mixer_alone(dev, layer):
    d = cfg_dict([layer], cap=0.0)
    m = build(d, dev)
    t = toks(37)
    r = HybridRunner(m, 64)
    close(r.step([("a", t)], all_rows(len(t))), oracle_logits(d, m, t), dev, layer["type"])


@pytest.mark.parametrize("dev", DEVICES)
def test_whole_model_with_loop_prefill_and_first_tokens(dev):
    m = build(FULL, dev)
    for n in (1, 2, 3, 33):  # the first tokens of a sequence, and a prompt across one key tile
        t = toks(n, seed=n)
        r = HybridRunner(m, 64)
        close(r.step([("a", t)], all_rows(n)), oracle_logits(FULL, m, t), dev, f"prompt of {n}")


@pytest.mark.parametrize("dev", DEVICES)
def test_residual_trace_matches_layer_runs(dev):
    m = build(FULL, dev)
    t = toks(9)
    W = {k: v.detach().cpu() for k, v in m.state_tensors().items()}
    want = []
    O.forward(FULL, W, t, torch.float64, want)
    pool = m.new_pool(1, 16)
    plan = BatchPlan.make([len(t)], [pool.alloc()], [0], m.device)
    got = []
    m(torch.tensor(t, dtype=torch.int32, device=m.device), plan, pool, trace=got)
    assert len(got) == len(want) == 7  # 1 + 2 * 2 + 2 layer runs
    for i, (g, w) in enumerate(zip(got, want)):
        close(g, w.float(), dev, f"stream after run {i}")


@pytest.mark.parametrize("dev", DEVICES)
def test_prefill_then_long_decode(dev):
    m = build(FULL, dev)
    t = toks(100, seed=3)
    want = oracle_logits(FULL, m, t)
    r = HybridRunner(m, 128)
    got = [r.step([("a", t[:30])], all_rows(30))]
    for p in range(30, 100):
        got.append(r.step([("a", [t[p]])]))
    close(torch.cat(got), want, dev, "decode")


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("cuts", [[2] * 20, [5, 2, 3, 1, 29], [31, 2, 7], [1, 1, 1, 37]], ids=str)
def test_portions_of_a_prompt(dev, cuts):
    m = build(FULL, dev)
    n = sum(cuts)
    t = toks(n, seed=5)
    want = oracle_logits(FULL, m, t)
    r = HybridRunner(m, 64)
    got, a = [], 0
    for c in cuts:
        got.append(r.step([("a", t[a:a + c])], all_rows(c)))
        a += c
    close(torch.cat(got), want, dev, f"cuts {cuts}")


@pytest.mark.parametrize("dev", DEVICES)
def test_unequal_batch_equals_each_alone_and_slots_are_reused(dev):
    m = build(FULL, dev)
    prompts = {"a": toks(1, seed=7), "b": toks(35, seed=8), "c": toks(12, seed=9)}
    tails = {k: toks(6, seed=20 + i) for i, k in enumerate(prompts)}
    want = {k: oracle_logits(FULL, m, prompts[k] + tails[k]) for k in prompts}
    r = HybridRunner(m, 64, n_slots=1)  # forces the pool to grow while the batch is built
    ids = list(prompts)
    out = r.step([(k, prompts[k]) for k in ids], [list(range(len(prompts[k]))) for k in ids])
    a = 0
    for k in ids:
        n = len(prompts[k])
        close(out[a:a + n], want[k][:n], dev, f"batched prompt {k}")
        a += n
    live = list(ids)
    for s in range(6):
        out = r.step([(k, [tails[k][s]]) for k in live])
        for row, k in enumerate(live):
            close(out[row:row + 1], want[k][len(prompts[k]) + s][None], dev, f"batched decode {k} step {s}")
        if s == 2:  # the shortest leaves early; the batch shrinks and its slot goes back
            r.end_sample("a")
            live.remove("a")
    # a new request takes the freed slot while others are live: it must start from zero state
    freed = r.pool.free_slots[0]
    t = toks(9, seed=33)
    got = r.step([("d", t)], all_rows(9))
    assert r.slots["d"] == freed
    close(got, oracle_logits(FULL, m, t), dev, "reused slot")
    for k in ("b", "c", "d"):
        r.end_sample(k)
    assert sorted(r.pool.free_slots) == list(range(r.pool.n_slots)) and not r.pool.length


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("taps", [1, 2])
def test_other_sizes_and_degenerate_values(dev, taps):
    delta = copy.deepcopy(DELTA)
    delta["mixer"].update(conv=taps, heads=2, kv_heads=2, dim=16, vdim=33)
    lat = copy.deepcopy(LATENT)
    lat["mixer"].update(heads=9, rot_dim=6, rot={"dims": 6, "base": 10000.0}, kv_rank=33, vdim=5)
    lat["mlp"] = None
    d = cfg_dict([delta, lat], loop={"start": 0, "stop": 2, "times": 1}, width=40, vocab=31)
    m = build(d, dev, ranks={"l0.mix.a1": 2, "l0.mix.g1": 7})
    t = toks(21, vocab=31, seed=4)
    want = oracle_logits(d, m, t)
    r = HybridRunner(m, 32)
    got = torch.cat([r.step([("a", t[:14])], all_rows(14))] + [r.step([("a", [x])]) for x in t[14:]])
    close(got, want, dev, f"taps {taps}")


@pytest.mark.parametrize("dev", DEVICES)
def test_far_key_dominates_attention(dev):
    """One key near the start of a long prompt is made to carry almost all the weight of the last query: scale its
    token's embedding so its rotated-key score stands out.  A kernel that loses far keys (or the first ones) fails."""
    lat = copy.deepcopy(LATENT)
    lat["mlp"] = None
    d = cfg_dict([lat], cap=0.0, vocab=400)
    m = build(d, dev)
    n = 300
    t = list(range(n))  # all tokens distinct
    for far in (0, 2, 31, 32, 150):
        emb = m.embed.data.clone()
        m.embed.data[t[far]] *= 6.0
        want = oracle_logits(d, m, t)
        r = HybridRunner(m, 512)
        got = torch.cat([r.step([("a", t[:-1])], all_rows(n - 1)), r.step([("a", t[-1:])])])
        close(got, want, dev, f"far key {far}")
        m.embed.data.copy_(emb)


@pytest.mark.parametrize("dev", DEVICES)
def test_recurrent_state_remembers_a_far_token(dev):
    """With decays pushed to ~1 the recurrences keep what an early token wrote; dropping or re-zeroing state between
    steps would change the logits hundreds of tokens later."""
    d = cfg_dict([GLA, DELTA], cap=0.0)
    m = build(d, dev)
    m.blocks[0].mix.a2_b.data.fill_(12.0)       # sigmoid(z)^(1/tau) ~ 1
    m.blocks[1].mix.A_log.data.fill_(-9.0)      # exp(-exp(A) softplus(.)) ~ 1
    t = toks(260, seed=11)
    want = oracle_logits(d, m, t)
    other = list(t)
    other[1] = (t[1] + 1) % 50
    assert (oracle_logits(d, m, other)[-1] - want[-1]).abs().max() > 50 * tol(dev) or dev[1] == torch.bfloat16
    r = HybridRunner(m, 300)
    got = torch.cat([r.step([("a", t[:200])], all_rows(200))] + [r.step([("a", [x])]) for x in t[200:]])
    close(got, want, dev, "far state")


@pytest.mark.parametrize("dev", DEVICES)
def test_greedy_generation_through_runner_and_pipeline_loop(dev):
    m = build(FULL, dev)
    prompts = [toks(5, seed=1), toks(11, seed=2)]
    ref = []
    for p in prompts:
        seq = list(p)
        for _ in range(6):
            seq.append(int(oracle_logits(FULL, m, seq)[-1].argmax()))
        ref.append(seq)
    r = HybridRunner(m, 32)
    out = r.generate(prompts, 6, SamplingParams.greedy())
    if dev[1] == torch.float32:
        assert out == ref
    assert not r.pool.length  # every slot returned
    # the recurrent-pipeline loop (one node, loopback ring) drives the same runner sample by sample
    running = threading.Event()
    running.set()
    res = starter_loop(HybridRunner(m, 32), LoopbackTransport(), [torch.tensor(p) for p in prompts], 6,
                       SamplingParams.greedy(), running, n_nodes=1)
    if dev[1] == torch.float32:
        assert [res.samples[i].view(-1).tolist() for i in range(2)] == ref


def test_checkpoint_roundtrip_registry_and_trace_cli(tmp_path):
    m = build(FULL, ("cpu", torch.float32))
    ck = tmp_path / "ck"
    ck.mkdir()
    m.config.save(ck)
    write_safetensors({k: v.to(torch.bfloat16) for k, v in m.state_tensors().items()}, ck / "model.safetensors")
    m2 = load_hybrid(ck, "cpu", torch.float32)
    t = toks(12)
    want = oracle_logits(FULL, m2, t)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": t[:8], "want": [0, 7]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": t[8:9], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": t[9:10], "want": [0]}, ], "end": ["x"]},
             {"step": 3, "entries": [{"id": "y", "tokens": t, "want": [11]}], "end": ["y"]}]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(ck), "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "16", "--device", "cpu"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    import numpy as np

    def rd(i):
        return torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, 50).copy())

    assert not (out / "1.f32").exists()
    close(rd(0), want[[0, 7]], ("cpu", torch.float32))
    close(rd(2), want[[9]], ("cpu", torch.float32))
    close(rd(3), want[[11]], ("cpu", torch.float32))


def test_config_validation_and_layer_runs():
    c = HybridConfig.from_dict(FULL)
    assert c.layer_runs() == [(0, False), (1, True), (2, False), (1, True), (2, False), (3, False), (4, False)]
    assert HybridConfig.from_dict(c.asdict()).layer_runs() == c.layer_runs()
    bad = copy.deepcopy(FULL)
    bad["layers"][0]["type"] = "nope"
    with pytest.raises(ValueError):
        HybridConfig.from_dict(bad)
    bad = copy.deepcopy(FULL)
    bad["loop"]["stop"] = 9
    with pytest.raises(ValueError):
        HybridConfig.from_dict(bad)
    with pytest.raises(ValueError):
        from mdi_llm_b200.models.registry import model_classes
        model_classes("unknown-arch")


def test_sequence_longer_than_pool_is_refused():
    m = build(cfg_dict([GLA]), ("cpu", torch.float32))
    r = HybridRunner(m, 8)
    with pytest.raises(ValueError):
        r.step([("a", toks(9))])


# ---- kernel variants against each other and against the PyTorch bodies (GPU only) --------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("shape", [(3, 1, 24, 20), (4, 4, 128, 128), (2, 1, 200, 64), (2, 2, 40, 300)], ids=str)
@pytest.mark.parametrize("mode", ["gla", "delta"])
def test_recurrence_kernels_agree(dtype, shape, mode):
    from mdi_llm_b200.ops import hybrid as H

    heads, kv, D, V = shape
    g = torch.Generator().manual_seed(0)
    lengths, starts = [5, 1, 17], [0, 0, 0]
    N = sum(lengths)

    def rnd(*s, scale=1.0):
        return (torch.randn(*s, generator=g) * scale).to(torch.bfloat16).float()

    t = dict(q=rnd(N, kv * D), k=rnd(N, kv * D), v=rnd(N, heads * V), z=rnd(N, heads * D), gate=rnd(N, heads * V),
             w=1 + rnd(V, scale=0.1), zb=rnd(heads * D), beta=rnd(N, heads), a_log=rnd(heads, scale=0.3))
    state0 = rnd(3, heads, D, V, scale=0.2)

    def run(device, dt, variant):
        x = {k: v.to(device=device, dtype=dt) for k, v in t.items()}
        st = state0.clone().to(device)
        plan = BatchPlan.make(lengths, [2, 0, 1], starts, torch.device(device))
        kw = dict(heads=heads, kv_heads=kv, dim=D, vdim=V, mode=mode, eps=1e-5, zb=x["zb"])
        if mode == "delta":
            kw.update(beta=x["beta"], a_log=x["a_log"])
        else:
            kw.update(tau=5.0)
        if device == "cuda":
            kw["variant"] = variant
        y = H.gated_recurrence(x["q"], x["k"], x["v"], x["z"], x["gate"], x["w"], st, plan, **kw)
        return y.float().cpu(), st.cpu()

    want_y, want_s = run("cpu", torch.float32, 0)
    variants = [1] + ([2] if (D <= 128 and V <= 128) or (D <= 256 and V <= 64) else [])
    variants += [3, 0]  # prepare / scan / finish kernels, and whatever the dispatcher picks for this step
    for variant in variants:
        y, s = run("cuda", dtype, variant)
        lim = 2e-4 if dtype == torch.float32 else 0.06
        assert (y - want_y).abs().max() < lim * max(1.0, want_y.abs().max().item()), f"variant {variant} output"
        assert (s - want_s).abs().max() < lim * max(1.0, want_s.abs().max().item()), f"variant {variant} state"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_split_key_attention_matches_unsplit_and_finds_one_far_key(dtype):
    from mdi_llm_b200.ops import hybrid as H

    Hh, D, R, L = 5, 16, 8, 40
    ctx = [700, 33, 1]
    g = torch.Generator().manual_seed(0)
    cache = (torch.randn(3, 704, L + R, generator=g) * 0.3).to(torch.bfloat16).float()
    qlat = (torch.randn(Hh, 3, L, generator=g) * 0.3).to(torch.bfloat16).float()
    q = (torch.randn(3, Hh * (D + R), generator=g) * 0.3).to(torch.bfloat16).float()
    # head 2 of sequence 0 looks for key 3: a copy of that key, scaled up, as its query
    qlat[2, 0] = cache[0, 3, :L] * 300
    plan_c = BatchPlan.make([1, 1, 1], [0, 1, 2], [c - 1 for c in ctx], torch.device("cpu"))
    want = H.latent_attn(qlat, q, cache, plan_c, Hh, D, R, L, 0.25)
    assert (want[2, 0] - cache[0, 3, :L]).abs().max() < 1e-2  # the far key really dominates
    plan = BatchPlan.make([1, 1, 1], [0, 1, 2], [c - 1 for c in ctx], torch.device("cuda"))
    args = [x.cuda().to(dtype) for x in (qlat, q, cache)]
    lim = 1e-5 if dtype == torch.float32 else 2e-2
    for split in (1, 0, 7, 32):
        got = H.latent_attn(args[0], args[1], args[2], plan, Hh, D, R, L, 0.25, split=split).float().cpu()
        assert (got - want).abs().max() < lim, f"split {split}"


@pytest.mark.parametrize("dev", DEVICES)
def test_expanded_prompt_attention_with_portions_and_query_blocks(dev, monkeypatch):
    """The prompt form of latent attention (keys and values expanded from the latents, scores in blocks of query
    rows) on portions that start in the middle of a sequence, with blocks that do not divide the portion."""
    from mdi_llm_b200.models.hybrid import LatentAttention

    monkeypatch.setattr(LatentAttention, "expand_from", 2)
    monkeypatch.setattr(LatentAttention, "query_block", 5)
    m = build(FULL, dev)
    cuts = [7, 12, 3, 1, 9]
    t = toks(sum(cuts), seed=6)
    want = oracle_logits(FULL, m, t)
    r = HybridRunner(m, 64)
    got, a = [], 0
    for c in cuts:
        got.append(r.step([("a", t[a:a + c])], all_rows(c)))
        a += c
    close(torch.cat(got), want, dev, "expanded form")
    # two prompts of different lengths in one step
    r2 = HybridRunner(m, 64)
    out = r2.step([("x", t[:20]), ("y", t[:9])], [list(range(20)), list(range(9))])
    close(out[:20], want[:20], dev, "batched x")
    close(out[20:], want[:9], dev, "batched y")
