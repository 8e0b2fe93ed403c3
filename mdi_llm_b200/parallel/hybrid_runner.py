"""Stage runner and batch scheduler of the hybrid model family.

:class:`HybridRunner` is a :class:`~.scheduler.StageRunner` (so the recurrent-pipeline loops of ``scheduler.py`` can
drive it one sample at a time, like any other stage) and adds what the transformer runners do not have: a *batched*
step.  ``step`` takes any number of live samples, each with the tokens it brings this step — whole prompts of
different lengths, or one token each — packs them into one token matrix without padding, and runs the model's step
function once against the sample's slots of the :class:`~..models.hybrid.StatePool`.  ``generate`` is the scheduler
on top: prompts are prefilled together, then every live sample advances one token per step; a sample that finishes
gives its slot back at once and the batch shrinks (no request joins a running batch).

On CUDA a one-token-per-sample step is replayed as a CUDA graph (one graph per batch size): the first step of a batch
size runs eagerly and warms the libraries up, the second is captured, later ones only refresh the token and
``{slot, position}`` tables on the device and replay.  Prompts always run eagerly.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..models.gpt import sample as sample_logits
from ..models.hybrid import HybridLM, StatePool
from ..ops.hybrid import BatchPlan
from .scheduler import SamplingParams, StageRunner

__all__ = ["HybridRunner"]


class _DecodeGraph:
    """Static inputs of a captured one-token step for ``n`` samples."""

    def __init__(self, n: int, device: torch.device) -> None:
        self.n = n
        self.host = torch.zeros(n, 5, dtype=torch.int32).pin_memory()  # token | row, count, slot, position
        self.tokens = torch.zeros(n, dtype=torch.int32, device=device)
        self.plan = BatchPlan.make([1] * n, [0] * n, [0] * n, device)
        self.graph = torch.cuda.CUDAGraph()
        self.logits: Optional[torch.Tensor] = None
        self.copied = torch.cuda.Event()

    def load(self, tokens: Sequence[int], slots: Sequence[int], pos: Sequence[int]) -> None:
        self.plan.seqs = [(i, 1, s, p) for i, (s, p) in enumerate(zip(slots, pos))]
        self.copied.synchronize()  # the previous step's copies have left the pinned buffer
        self.host.copy_(torch.tensor([[t, i, 1, s, p] for i, (t, s, p) in enumerate(zip(tokens, slots, pos))], dtype=torch.int32))
        self.tokens.copy_(self.host[:, 0], non_blocking=True)
        self.plan.meta.copy_(self.host[:, 1:], non_blocking=True)
        self.copied.record()


class HybridRunner(StageRunner):
    role = "starter"

    def __init__(self, model: HybridLM, max_seq_length: int, n_slots: int = 4, use_graphs: Optional[bool] = None) -> None:
        self.model = model.eval()
        self.device, self.dtype = model.device, model.dtype
        self.pool: StatePool = model.new_pool(n_slots, max_seq_length)
        self.slots: Dict[object, int] = {}
        self.use_graphs = self.device.type == "cuda" if use_graphs is None else bool(use_graphs)
        self._graphs: Dict[int, "_DecodeGraph"] = {}
        self._seen: Dict[int, int] = {}
        self._pool_slots = self.pool.n_slots

    # ---- sample life cycle -----------------------------------------------------------------------
    def begin_sample(self, sample_id: object) -> None:
        if sample_id not in self.slots:
            self.slots[sample_id] = self.pool.alloc()

    def end_sample(self, sample_id: object) -> None:
        self.pool.free(self.slots.pop(sample_id))

    def position(self, sample_id: object) -> int:
        return self.pool.length[self.slots[sample_id]]

    # ---- batched step ----------------------------------------------------------------------------
    def _plan(self, entries: Sequence[Tuple[object, Sequence[int]]]) -> Tuple[torch.Tensor, BatchPlan]:
        ids = [sid for sid, _ in entries]
        if len(set(ids)) != len(ids):
            raise ValueError("a sample appears twice in one step")
        for sid in ids:
            self.begin_sample(sid)
        slots = [self.slots[sid] for sid in ids]
        lengths = [len(t) for _, t in entries]
        if min(lengths, default=1) < 1:
            raise ValueError("every entry of a step brings at least one token")
        plan = BatchPlan.make(lengths, slots, [self.pool.length[s] for s in slots], self.device)
        flat = [int(t) for _, toks in entries for t in toks]
        tokens = torch.tensor(flat, dtype=torch.int32).to(self.device)
        return tokens, plan

    def _advance(self, plan: BatchPlan) -> None:
        for _, n, slot, p0 in plan.seqs:
            self.pool.length[slot] = p0 + n

    @torch.inference_mode()
    def step(self, entries: Sequence[Tuple[object, Sequence[int]]],
             want: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """Run one step. ``want[i]`` lists the places among entry i's tokens whose logits are returned (default: its
        last token); the result is fp32 ``[sum of wanted, vocab]`` in entry order."""
        if self.use_graphs and entries and all(len(t) == 1 for _, t in entries):
            out = self._graph_step(entries)
            if out is not None:
                if want is None or all(len(w) == 1 for w in want):
                    return out
                keep = [i for i, w in enumerate(want) if len(w)]
                return out.index_select(0, torch.tensor(keep, dtype=torch.long, device=self.device))
        tokens, plan = self._plan(entries)
        if want is None:
            rows = plan.last_rows
        else:
            rows = [r0 + int(w) for (r0, _, _, _), ws in zip(plan.seqs, want) for w in ws]
        x = self.model.hidden(tokens, plan, self.pool)
        self._advance(plan)
        if not rows:
            return torch.empty(0, self.model.config.vocab, device=self.device)
        return self.model.head(x.index_select(0, torch.tensor(rows, dtype=torch.long, device=self.device)))

    def _graph_step(self, entries: Sequence[Tuple[object, Sequence[int]]]) -> Optional[torch.Tensor]:
        """One token per sample through a captured graph; None while this batch size is still warming up."""
        n = len(entries)
        ids = [sid for sid, _ in entries]
        if len(set(ids)) != n:
            raise ValueError("a sample appears twice in one step")
        for sid in ids:
            self.begin_sample(sid)
        if self.pool.n_slots != self._pool_slots:  # the pool grew: its tensors moved, captured graphs are void
            self._graphs.clear()
            self._pool_slots = self.pool.n_slots
        slots = [self.slots[sid] for sid in ids]
        pos = [self.pool.length[s] for s in slots]
        if max(pos) + 1 > self.pool.max_seq_length:
            raise ValueError(f"sequence exceeds the pool's max_seq_length {self.pool.max_seq_length}")
        g = self._graphs.get(n)
        if g is None:
            self._seen[n] = self._seen.get(n, 0) + 1
            if self._seen[n] < 2:
                return None
            g = _DecodeGraph(n, self.device)
            g.load([int(t[0]) for _, t in entries], slots, pos)
            torch.cuda.synchronize(self.device)
            with torch.cuda.graph(g.graph):
                g.logits = self.model.head(self.model.hidden(g.tokens, g.plan, self.pool))
            self._graphs[n] = g
        g.load([int(t[0]) for _, t in entries], slots, pos)
        g.graph.replay()
        self._advance(g.plan)
        return g.logits.clone()  # the graph's output buffer is overwritten by the next replay

    # ---- StageRunner interface (one sample per call) ----------------------------------------------
    @torch.inference_mode()
    def forward(self, sample_id: int, data: torch.Tensor, input_pos: Optional[torch.Tensor]) -> torch.Tensor:
        if input_pos is None:
            raise NotImplementedError("hybrid models carry recurrent state: a cache-less forward does not exist")
        toks = data.view(-1).tolist()
        if int(input_pos[0]) != self.position(sample_id):
            raise ValueError(f"sample {sample_id} is at position {self.position(sample_id)}, got {int(input_pos[0])}")
        tokens, plan = self._plan([(sample_id, toks)])
        x = self.model.hidden(tokens, plan, self.pool)
        self._advance(plan)
        return x.unsqueeze(0)

    @torch.inference_mode()
    def head(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.model.head(hidden[0, -1:].float().contiguous()).unsqueeze(0)

    # ---- scheduler ---------------------------------------------------------------------------------
    @torch.inference_mode()
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int, sampling: Optional[SamplingParams] = None,
                 stop_token: Optional[int] = None, on_token: Optional[Callable[[int, int], None]] = None) -> List[List[int]]:
        """Continue every prompt by up to ``max_new_tokens`` tokens; returns prompt + continuation per sample."""
        sampling = sampling or SamplingParams.greedy()
        gen = None
        if sampling.seed is not None:
            gen = torch.Generator(device="cpu").manual_seed(sampling.seed)
        out = [list(map(int, p)) for p in prompts]
        live = list(range(len(out)))
        base = object()
        ids = {i: (base, i) for i in live}
        entries = [(ids[i], out[i]) for i in live]
        for _ in range(max_new_tokens):
            logits = self.step(entries)
            nxt: List[Tuple[int, int]] = []
            for row, i in enumerate(live):
                lg = logits[row].float()
                tok = int(sample_logits(lg.cpu() if gen is not None else lg, temperature=sampling.temperature,
                                        top_k=sampling.top_k, top_p=sampling.top_p, generator=gen))
                out[i].append(tok)
                if on_token is not None:
                    on_token(i, tok)
                if stop_token is not None and tok == stop_token:
                    self.end_sample(ids[i])
                else:
                    nxt.append((i, tok))
            live = [i for i, _ in nxt]
            entries = [(ids[i], [tok]) for i, tok in nxt]
            if not live:
                break
        for i in live:
            self.end_sample(ids[i])
        return out
