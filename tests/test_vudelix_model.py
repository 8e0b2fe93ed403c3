"""The Vudelix design (pre-norm blocks of the hybrid family) against the plain oracle of ``vudelix_oracle.py``.

Every test builds its own small configuration with random weights.  Sizes are awkward on purpose: value width != key
width, several query heads per key head and exactly one, rotary on part of a head and on all of it, frequency
stretching that hits all three of its branches, a window shorter than every prompt and one longer than any, one and
several experts per token, a layer without feed-forward, a model without the per-layer token embedding.  The same
tests run on the CPU (PyTorch bodies of the operations) and, marked ``gpu``, on the sm_100a kernels.
"""
from __future__ import annotations

import copy
import json
import os
import subprocess
import sys

import pytest
import torch

import vudelix_oracle as O
from mdi_llm_b200.models.config import HybridConfig
from mdi_llm_b200.models.hybrid import HybridLM, MoEFF, WindowAttention, load_hybrid, write_safetensors
from mdi_llm_b200.models.registry import model_classes
from mdi_llm_b200.ops import hybrid as H
from mdi_llm_b200.ops.hybrid import BatchPlan
from mdi_llm_b200.parallel.hybrid_runner import HybridRunner
from mdi_llm_b200.parallel.scheduler import SamplingParams

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

MOE = {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 2}}
ATT = {"type": "attention", "mlp": MOE,
       "mixer": {"heads": 6, "kv_heads": 2, "dim": 12, "vdim": 10, "scale": 0.4, "mask": {"size": 7},
                 "rot": {"dims": 8, "base": 50.0, "scaling": {"factor": 3.0, "low": 1.0, "high": 4.0, "original": 32}}}}
ATT_WIDE = {"type": "attention", "mlp": {"kind": "dense", "ff": 40},
            "mixer": {"heads": 3, "kv_heads": 3, "dim": 8, "vdim": 16, "scale": 1.5, "mask": {"size": 500},
                      "rot": {"dims": 8, "base": 10000.0}}}
DELTA = {"type": "channel_delta", "mlp": {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 3, "top": 1}},
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 10, "conv": 4}}
DELTA_BARE = {"type": "channel_delta", "mlp": None, "mixer": {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 8, "conv": 2}}


def cfg_dict(layers, width=24, vocab=50, mult=0.7, side=6):
    d = {"architecture": "Vudelix", "vocab": vocab, "width": width, "layers": copy.deepcopy(layers),
         "norm": {"eps": 1e-5}, "residual_mult": mult}
    if side:
        d["token_side"] = {"dim": side}
    return d


def all_experts(d):
    """The same model with every expert chosen for every token: no routing decision that 8-bit mantissas could flip."""
    d = copy.deepcopy(d)
    for spec in d["layers"]:
        if spec["mlp"] and spec["mlp"]["kind"] == "moe":
            spec["mlp"]["router"]["top"] = spec["mlp"]["router"]["experts"]
    return d


FULL = cfg_dict([DELTA, ATT, DELTA_BARE, ATT_WIDE])

DEVICES = [pytest.param(("cpu", torch.float32), id="cpu-f32"),
           pytest.param(("cuda", torch.float32), id="cuda-f32", marks=pytest.mark.gpu),
           pytest.param(("cuda", torch.bfloat16), id="cuda-bf16", marks=pytest.mark.gpu)]


def build(d, dev, seed=0):
    device, dtype = dev
    if device == "cuda":
        torch.backends.cuda.matmul.allow_tf32 = False
    if dtype == torch.bfloat16:
        d = all_experts(d)
    ranks = {f"l{i}.mix.{n}": r for i in range(len(d["layers"])) for n, r in (("a1", 5), ("g1", 3))}
    return d, HybridLM(HybridConfig.from_dict(d), ranks).init_random(device, dtype, seed)


def oracle_logits(d, model, tokens, trace=None):
    W = {k: v.detach().cpu() for k, v in model.state_tensors().items()}
    return O.forward(d, W, list(tokens), torch.float64, trace).float()


def close(got, want, dev, what=""):
    """fp32: every value within 2e-4.  bf16: per row, the error (root mean square over the row) relative to the row's
    own spread is below 8 % on average and 40 % at the worst row (models this narrow average a rounding error over
    few terms)."""
    diff = got.float().cpu() - want
    if dev[1] == torch.float32:
        err = diff.abs().max().item()
        assert err < 2e-4, f"{what}: max abs error {err}"
        return
    rel = diff.pow(2).mean(-1).sqrt() / want.std(-1).clamp_min(1e-3)
    assert rel.mean().item() < 0.08 and rel.max().item() < 0.4, f"{what}: relative rms error mean {rel.mean()} max {rel.max()}"


def toks(n, vocab=50, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def all_rows(n):
    return [list(range(n))]


# ---- each mechanism alone -----------------------------------------------------------------------------------
@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("case", ["attention", "attention_wide", "attention_unbounded", "delta", "moe", "side", "no_side_no_mult"])
def test_each_mechanism_alone(dev, case):
    bare = lambda spec: {**copy.deepcopy(spec), "mlp": None}
    plain = {"type": "attention", "mlp": None, "mixer": {"heads": 1, "kv_heads": 1, "dim": 6, "vdim": 4, "scale": 0.9}}
    d = {"attention": cfg_dict([bare(ATT)], side=0), "attention_unbounded": cfg_dict([plain, plain], side=0), "attention_wide": cfg_dict([bare(ATT_WIDE)], side=0),
         "delta": cfg_dict([DELTA_BARE], side=0), "moe": cfg_dict([{**copy.deepcopy(DELTA_BARE), "mlp": MOE}], side=0),
         "side": cfg_dict([DELTA_BARE], side=5), "no_side_no_mult": cfg_dict([ATT_WIDE], side=0, mult=1.0)}[case]
    d, m = build(d, dev)
    t = toks(41)
    close(HybridRunner(m, 64).step([("a", t)], all_rows(len(t))), oracle_logits(d, m, t), dev, case)


def test_stretched_frequencies_take_all_three_branches():
    rot = ATT["mixer"]["rot"]
    plain = O.stretched_frequencies(rot["dims"], rot["base"], None)
    got = H.scaled_inv_freq(rot["dims"], rot["base"], rot["scaling"], torch.device("cpu")).tolist()
    want = O.stretched_frequencies(rot["dims"], rot["base"], rot["scaling"])
    assert got == pytest.approx(want, rel=1e-6)
    ratio = [w / p for w, p in zip(want, plain)]
    assert ratio[0] == 1.0 and ratio[-1] == pytest.approx(1 / 3) and 1 / 3 < ratio[1] < 1.0


def test_router_picks_largest_scores_lower_index_on_ties():
    z = torch.tensor([[0.1, 2.0, 2.0, -1.0], [3.0, -2.0, 0.5, 0.5]])
    idx, wt = H.router_topk(z, 3)
    assert idx.tolist() == [[1, 2, 0], [0, 2, 3]]
    assert torch.allclose(wt, torch.sigmoid(torch.tensor([[2.0, 2.0, 0.1], [3.0, 0.5, 0.5]])))


@pytest.mark.gpu
def test_router_kernel_matches():
    z = torch.randn(300, 9, generator=torch.Generator().manual_seed(0))
    z[5, 3] = z[5, 7] = 9.0
    for top in (1, 4, 9):
        i0, w0 = H.router_topk(z, top)
        i1, w1 = H.router_topk(z.cuda(), top)
        assert torch.equal(i0, i1.cpu()) and torch.allclose(w0, w1.cpu(), atol=1e-6)


# ---- prompts, decoding, portions, batches -------------------------------------------------------------------
@pytest.mark.parametrize("dev", DEVICES)
def test_whole_prompts_and_first_tokens(dev, monkeypatch):
    monkeypatch.setattr(WindowAttention, "query_block", 48)
    d, m = build(FULL, dev)
    for n in (1, 2, 3, 7, 8, 70, 150):  # the first tokens; the short window's edge; one band; several bands
        t = toks(n, seed=n)
        close(HybridRunner(m, 160).step([("a", t)], all_rows(n)), oracle_logits(d, m, t), dev, f"prompt of {n}")


@pytest.mark.parametrize("dev", DEVICES)
def test_residual_trace(dev):
    d, m = build(FULL, dev)
    t = toks(9)
    want = []
    oracle_logits(d, m, t, want)
    pool = m.new_pool(1, 16)
    plan = BatchPlan.make([len(t)], [pool.alloc()], [0], m.device)
    got = []
    m(torch.tensor(t, dtype=torch.int32, device=m.device), plan, pool, trace=got)
    assert len(got) == len(want) == 4
    for i, (g, w) in enumerate(zip(got, want)):
        close(g, w.float(), dev, f"stream after layer {i}")


@pytest.mark.parametrize("dev", DEVICES)
def test_prefill_then_long_decode(dev):
    d, m = build(FULL, dev)
    t = toks(110, seed=3)
    want = oracle_logits(d, m, t)
    r = HybridRunner(m, 128)
    got = [r.step([("a", t[:30])], all_rows(30))]
    for p in range(30, 110):  # the short window slides past the whole prompt many times over
        got.append(r.step([("a", [t[p]])]))
    close(torch.cat(got), want, dev, "decode")
    # token by token from the very first token equals the prompt form
    r2 = HybridRunner(m, 128)
    one = torch.cat([r2.step([("b", [x])]) for x in t[:20]])
    close(one, want[:20], dev, "token by token")


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("cuts", [(2, 3, 2, 64, 5, 70, 1, 2, 11), (66, 2, 92), (160,)], ids=["small", "mixed", "whole"])
def test_portions_of_a_prompt(dev, cuts, monkeypatch):
    monkeypatch.setattr(WindowAttention, "query_block", 40)
    d, m = build(FULL, dev)
    t = toks(sum(cuts), seed=5)
    want = oracle_logits(d, m, t)
    r = HybridRunner(m, 192)
    got, at = [], 0
    for c in cuts:
        got.append(r.step([("a", t[at:at + c])], all_rows(c)))
        at += c
    close(torch.cat(got), want, dev, f"portions {cuts}")


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("lengths", [(5, 19, 1, 9), (70, 64, 90)], ids=["short", "banded"])
def test_unequal_batch_equals_each_alone_and_slots_are_reused(dev, lengths):
    d, m = build(FULL, dev)
    seqs = {f"s{i}": toks(n + 12, seed=10 + i) for i, n in enumerate(lengths)}
    want = {k: oracle_logits(d, m, v) for k, v in seqs.items()}
    r = HybridRunner(m, 128, n_slots=2)  # the pool has to grow
    live = list(seqs)
    out = r.step([(k, seqs[k][:n]) for k, n in zip(live, lengths)], [list(range(n)) for n in lengths])
    at = 0
    for k, n in zip(live, lengths):
        close(out[at:at + n], want[k][:n], dev, f"prompt {k}")
        at += n
    pos = dict(zip(live, lengths))
    for stepno in range(12):
        if stepno == 4:  # one request ends early; its slot goes back
            r.end_sample(live.pop(1))
        out = r.step([(k, [seqs[k][pos[k]]]) for k in live])
        for i, k in enumerate(live):
            close(out[i:i + 1], want[k][pos[k]:pos[k] + 1], dev, f"decode {k} at {pos[k]}")
            pos[k] += 1
    for k in live:
        r.end_sample(k)
    assert not r.pool.length
    # freed slots serve a new request: nothing of the old state or cache shows
    t = toks(75, seed=99)
    close(r.step([("new", t)], all_rows(75)), oracle_logits(d, m, t), dev, "reused slot")


@pytest.mark.parametrize("dev", DEVICES)
def test_greedy_generation_through_the_runner(dev):
    d, m = build(FULL, dev)
    prompts = [toks(5, seed=1), toks(11, seed=2)]
    r = HybridRunner(m, 32)
    out = r.generate(prompts, 6, SamplingParams.greedy())
    assert not r.pool.length
    if dev[1] == torch.float32:
        for p, o in zip(prompts, out):
            seq = list(p)
            for _ in range(6):
                seq.append(int(oracle_logits(d, m, seq)[-1].argmax()))
            assert o == seq


# ---- window edges and far keys: one score made to stand out -------------------------------------------------
def _sharp_case(dev, W, S=160, G=2, rep=3, D=8, V=6):
    """A cache of unit keys and random values, and for every position four queries (one per target) that point
    at one chosen key with a large score: the key just inside the window, the one just outside, the first key of
    the sequence, and the token itself."""
    device, dtype = dev
    g = torch.Generator().manual_seed(4)
    k = torch.nn.functional.normalize(torch.randn(S, G, D, generator=g), dim=-1)
    v = torch.randn(S, G, V, generator=g)
    cache = torch.zeros(2, S, G * (D + V))
    cache[1, :, :G * D] = k.reshape(S, -1)
    cache[1, :, G * D:] = v.reshape(S, -1)
    return k, v, cache.to(device=device, dtype=dtype)


def _plain_window(q, k, v, pos, W, scale, rep):
    """q [H, D] at position pos over keys k [S, G, D], values v [S, G, V]; plain loops."""
    H_ = q.shape[0]
    first = max(0, pos - W + 1)
    out = []
    for h in range(H_):
        g = h // rep
        s = torch.stack([(q[h] @ k[j, g]) * scale for j in range(first, pos + 1)])
        w = torch.softmax(s, 0)
        out.append(sum(w[j - first] * v[j, g] for j in range(first, pos + 1)))
    return torch.cat(out)


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("W", [5, 33, 64])
def test_keys_just_inside_and_outside_the_window_and_far_back(dev, W, monkeypatch):
    monkeypatch.setattr(WindowAttention, "query_block", 32)
    device, dtype = dev
    G, rep, D, V, S = 2, 3, 8, 6, 160
    Hh = G * rep
    k, v, cache = _sharp_case(dev, W)
    kq, vq = (k.to(dtype).float(), v.to(dtype).float())
    for target in ("inside", "outside", "first", "self"):
        pick = {"inside": lambda p: max(0, p - W + 1), "outside": lambda p: max(0, p - W), "first": lambda p: 0,
                "self": lambda p: p}[target]
        q = torch.stack([20.0 * k[pick(p)].repeat_interleave(rep, 0) for p in range(S)]).to(dtype)  # [S, H, D]
        qf = q.float()
        want = torch.stack([_plain_window(qf[p], kq, vq, p, W, 1.0, rep) for p in range(S)])
        qd = q.reshape(S, Hh * D).to(device)
        # decoding: one token per step at positions around the edges
        for p in (0, 1, W - 1, W, W + 1, 2 * W, S - 1):
            plan = BatchPlan.make([1], [1], [p], torch.device(device))
            got = H.window_attn(qd[p:p + 1].contiguous(), None, cache, plan, Hh, G, D, V, 1.0, W)
            assert (got.float().cpu() - want[p]).abs().max() < (1e-4 if dtype == torch.float32 else 0.05), (target, p)
        # a portion of a prompt that starts in the middle, in both forms
        p0, n = 37, 100
        plan = BatchPlan.make([n], [1], [p0], torch.device(device))
        got = H.window_attn(qd[p0:p0 + n].contiguous(), None, cache, plan, Hh, G, D, V, 1.0, W)
        assert (got.float().cpu() - want[p0:p0 + n]).abs().max() < (1e-4 if dtype == torch.float32 else 0.05), target
        att = WindowAttention(16, {"heads": Hh, "kv_heads": G, "dim": D, "vdim": V, "scale": 1.0, "mask": {"size": W}}, 1e-5)
        band = att._banded(qd[p0:p0 + n].contiguous(), cache, plan)  # [H, n, V]
        got = band.permute(1, 0, 2).reshape(n, Hh * V)
        assert (got.float().cpu() - want[p0:p0 + n]).abs().max() < (1e-4 if dtype == torch.float32 else 0.05), target
    # the target outside the window must not be what the output shows: its value is far from the result
    p = 2 * W
    plan = BatchPlan.make([1], [1], [p], torch.device(device))
    q = (20.0 * k[p - W].repeat_interleave(rep, 0)).reshape(1, -1).to(device=device, dtype=dtype)
    got = H.window_attn(q, None, cache, plan, Hh, G, D, V, 1.0, W).float().cpu().view(Hh, V)
    assert (got[0] - v[p - W, 0]).abs().max() > 0.2


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_key_shares_of_the_decode_form_agree(dtype):
    G, rep, D, V, S, W = 2, 3, 8, 6, 160, 70
    k, v, cache = _sharp_case(("cuda", dtype), W)
    g = torch.Generator().manual_seed(1)
    q = torch.randn(3, G * rep * D, generator=g).to(device="cuda", dtype=dtype)
    gate = torch.randn(3, G * rep, generator=g).to(device="cuda", dtype=dtype)
    plan = BatchPlan.make([1, 1, 1], [1, 1, 1], [3, 69, 159], torch.device("cuda"))
    one = H.window_attn(q, gate, cache, plan, G * rep, G, D, V, 0.8, W, split=1)
    for split in (0, 2, 5):  # 5 shares: some get no tile at all for the short context
        got = H.window_attn(q, gate, cache, plan, G * rep, G, D, V, 0.8, W, split=split)
        assert (got.float() - one.float()).abs().max() < (1e-5 if dtype == torch.float32 else 0.02), split


@pytest.mark.parametrize("dev", DEVICES)
def test_append_rotates_normalises_and_writes_the_cache(dev):
    device, dtype = dev
    Hh, G, D, V, nrot, eps = 4, 2, 10, 6, 6, 1e-5
    g = torch.Generator().manual_seed(2)
    N = 9
    q, k, v = torch.randn(N, Hh * D, generator=g), torch.randn(N, G * D, generator=g), torch.randn(N, G * V, generator=g)
    freqs = O.stretched_frequencies(nrot, 30.0, None)
    plan = BatchPlan.make([4, 5], [2, 0], [3, 0], torch.device(device))
    cache = torch.zeros(3, 12, G * (D + V), device=device, dtype=dtype)
    qd = q.to(device=device, dtype=dtype).clone()
    H.window_append(qd, k.to(device=device, dtype=dtype), v.to(device=device, dtype=dtype),
                    H.scaled_inv_freq(nrot, 30.0, None, torch.device(device)), cache, plan, Hh, G, D, V, nrot, eps)
    tol = 1e-5 if dtype == torch.float32 else 0.03
    qr, kr = q.to(dtype).double(), k.to(dtype).double()
    for row, (slot, pos) in enumerate([(2, 3), (2, 4), (2, 5), (2, 6), (0, 0), (0, 1), (0, 2), (0, 3), (0, 4)]):
        for h in range(Hh):
            want = O.rms_norm(O.rotate_neighbours(qr[row, h * D:(h + 1) * D], pos, freqs), None, eps)
            assert (qd[row, h * D:(h + 1) * D].double().cpu() - want).abs().max() < tol
        for h in range(G):
            want = O.rms_norm(O.rotate_neighbours(kr[row, h * D:(h + 1) * D], pos, freqs), None, eps)
            assert (cache[slot, pos, h * D:(h + 1) * D].double().cpu() - want).abs().max() < tol
        assert torch.equal(cache[slot, pos, G * D:].cpu(), v[row].to(dtype))
    assert cache[1].abs().sum() == 0 and cache[2, :3].abs().sum() == 0  # rows of other slots and positions untouched


# ---- mixture of experts: the two forms against a plain loop -------------------------------------------------
@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("sizes", [(40, 24, 6, 3), (33, 18, 4, 1), (7, 8, 2, 2)], ids=["top3", "top1", "all"])
def test_expert_forms_agree_with_a_plain_loop(dev, sizes, monkeypatch):
    device, dtype = dev
    C, ff, E, top = sizes
    g = torch.Generator().manual_seed(7)
    moe = MoEFF(C, ff, E, top)
    for p in moe.parameters():
        p.data = (torch.randn(p.shape, generator=g) * p.shape[-1] ** -0.5).to(device=device, dtype=dtype)
    moe.finalize()
    N = 50
    h = torch.randn(N, C, generator=g).to(device=device, dtype=dtype)
    idx, wt = H.router_topk(H.linear_f32(h, moe.router32), top)
    want = torch.zeros(N, C, dtype=torch.float64)
    for t in range(N):
        for j in range(top):
            e = int(idx[t, j])
            a = torch.relu(moe.e_up[e].double().cpu() @ (wt[t, j].double().cpu() * h[t].double().cpu())) ** 2
            want[t] += moe.e_down[e].double().cpu() @ a
    tol = 1e-4 if dtype == torch.float32 else 0.08
    monkeypatch.setattr(MoEFF, "gemv_max", 10 ** 6)
    a = moe(h)
    monkeypatch.setattr(MoEFF, "gemv_max", 0)
    b = moe(h)
    for got, what in ((a, "index-driven"), (b, "grouped")):
        assert (got.double().cpu() - want).abs().max() < tol * max(1.0, want.abs().max().item()), what
    # a token's result does not depend on its neighbours in the batch
    monkeypatch.setattr(MoEFF, "gemv_max", 10 ** 6)
    assert torch.equal(moe(h[3:4]), a[3:4])


# ---- checkpoint, registry, command line ---------------------------------------------------------------------
def test_checkpoint_roundtrip_registry_and_trace_cli(tmp_path):
    d, m = build(FULL, ("cpu", torch.float32))
    ck = tmp_path / "ck"
    ck.mkdir()
    m.config.save(ck)
    write_safetensors({k: v.to(torch.bfloat16) for k, v in m.state_tensors().items()}, ck / "model.safetensors")
    cfg_cls, model_cls = model_classes("Vudelix")
    assert cfg_cls is HybridConfig and model_cls is HybridLM
    m2 = load_hybrid(ck, "cpu", torch.float32)
    assert m2.config.block == "prenorm" and m2.config.norm == "rms" and m2.head_w is not None
    assert m2.config.residual_mult == 0.7 and m2.config.token_side == {"dim": 6}
    t = toks(12)
    want = oracle_logits(d, m2, t)
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


def test_config_validation():
    with pytest.raises(ValueError):
        HybridConfig.from_dict(cfg_dict([{**copy.deepcopy(ATT), "mlp": {"kind": "sparse"}}]))
    with pytest.raises(ValueError):
        HybridConfig.from_dict(cfg_dict([{**copy.deepcopy(ATT), "mlp": {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 2, "top": 3}}}]))
    bad = copy.deepcopy(ATT)
    bad["mixer"]["kv_heads"] = 4
    with pytest.raises(ValueError):
        HybridConfig.from_dict(cfg_dict([bad]))
    c = HybridConfig.from_dict(cfg_dict([ATT_WIDE], side=0, mult=1.0))
    assert c.token_side is None and c.residual_mult == 1.0 and not c.tied_head
    assert HybridConfig.from_dict(c.asdict()).asdict() == c.asdict()
