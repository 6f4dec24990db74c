"""Paged-KV autoregressive generation with continuous batching and CUDA-graph decode steps.

Design (B200-first):
  * KV lives in fixed pages of 64 tokens; a row reserves the pages for its longest possible
    sequence when it is admitted and gives them back when it finishes, so the page table of a slot
    never changes while the row runs and finished rows never trigger the compaction copies the
    reference performs per layer (RPEG/runtime/workers/megatron_worker.py:2585-2598).
  * One decode step (all layers, LM head, sampling, state advance) is captured once per slot-count
    bucket as a CUDA graph and replayed; positions, tokens, EOS detection and output recording are
    advanced on the device, so the host only looks at a finished-row counter every few steps.
  * When rows finish, queued prompts are prefilled into the free slots (continuous batching); when
    the queue is empty and few rows remain, live slots are compacted to the front and a smaller
    bucket graph takes over. Because KV is paged, compaction moves page-table rows, not KV.
  * Sampling log-probs are recorded as the PPO/GRPO ``old_logps`` (no second forward), as in the
    reference (megatron_worker.py:2493-2505).
Semantics kept from the reference's quantile-phase generation (:2370-2628): rows end at EOS or at
the length cap; outputs are returned per original row index, right padded, with a response mask.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..models.llama import LlamaModel
from ..ops import _lib
from ..ops import kernels as K

PAGE = K.KV_PAGE


class PagePool:
    """Host-side free list of KV pages. Page 0 is a scratch page retired slots point at."""

    def __init__(self, num_pages: int):
        if num_pages < 2:
            raise ValueError("need at least two KV pages")
        self.num_pages = num_pages
        self.free: List[int] = list(range(num_pages - 1, 0, -1))

    def available(self) -> int:
        return len(self.free)

    def take(self, n: int) -> List[int]:
        if n > len(self.free):
            raise RuntimeError(f"KV page pool exhausted: want {n}, have {len(self.free)}")
        out = self.free[-n:]
        del self.free[-n:]
        return out

    def give(self, pages: List[int]) -> None:
        self.free.extend(pages)


@dataclass
class GenerationResult:
    tokens: torch.Tensor        # [N, max_new] int32, right padded with pad_id
    logprobs: torch.Tensor      # [N, max_new] fp32 log-prob of each generated token under the sampling policy
    lengths: torch.Tensor       # [N] int32 number of generated tokens (EOS included)
    counters: Dict[str, float] = field(default_factory=dict)

    def response_mask(self) -> torch.Tensor:
        t = torch.arange(self.tokens.shape[1], device=self.tokens.device)
        return (t[None, :] < self.lengths[:, None]).float()


class Generator:
    BUCKETS = (256, 192, 128, 96, 64, 48, 32, 24, 16, 8)
    PDL_MAX_BATCH = 64
    GROUP_MAX = 8              # queries the group attention kernel scores per K/V tile
    GROUP_MIN_BATCH = 128      # the group kernel is one more launch per layer: it pays only while many rows are live
    GROUP_MIN = 3              # smaller groups are cheaper row by row

    @staticmethod
    def kv_bytes_for(cfg, slots: int, max_seq_len: int, tp: int = 1) -> int:
        """Bytes of KV storage that ``slots`` rows of up to ``max_seq_len`` tokens need (+ scratch page) on one of
        ``tp`` tensor-parallel ranks (each keeps its own KV heads)."""
        pages = slots * ((max_seq_len + PAGE - 1) // PAGE) + 1
        return 2 * cfg.n_layers * pages * (cfg.n_kv_heads // tp) * PAGE * cfg.head_dim * 2

    def __init__(self, model: LlamaModel, *, max_slots: int = 64, max_seq_len: int = 2048, kv_budget_bytes: float = 16e9,
                 eos_id: int = 2, pad_id: int = 0, sync_interval: int = 8, use_graphs: bool = True,
                 kv_storage: Optional[torch.Tensor] = None, group_attention: bool = False):
        """``kv_storage``: optional flat bf16 tensor to carve the KV pages from instead of allocating
        them; lets the cache share memory with buffers that are dead during generation (gradients)."""
        cfg = model.cfg
        self.model, self.cfg, self.dev = model, cfg, model.device
        # a tensor-parallel model (models.tp_decode.TPDecodeModel) keeps only its own heads in the cache
        # with peers in the decode step a lost rank must end the loop at the next host sync, not at the length cap
        self.check_status_every_sync = getattr(model, "tp", 1) > 1
        self.n_kv = getattr(model, "n_kv_local", cfg.n_kv_heads)
        self.n_heads = getattr(model, "n_heads_local", cfg.n_heads)
        self.eos_id, self.pad_id = eos_id, pad_id
        # rows that alias a prompt's KV pages are attended to as a group: the shared keys are read once per group.
        # ``True`` / ``"cuda"``: the CUDA-core group kernel; ``"tc"``: the tcgen05 one (keys on the M axis).
        self.group_attention = bool(group_attention) and not cfg.qk_norm
        self.group_tc = str(group_attention).lower() == "tc"
        self.group_min_batch = self.GROUP_MIN_BATCH
        self.sync_interval = max(1, sync_interval)
        self.use_graphs = use_graphs
        self.max_seq_len = max_seq_len
        self.pages_per_row = (max_seq_len + PAGE - 1) // PAGE
        page_bytes = 2 * cfg.n_layers * self.n_kv * PAGE * cfg.head_dim * 2
        if kv_storage is not None:
            kv_budget_bytes = kv_storage.numel() * 2
        num_pages = min(int(kv_budget_bytes // page_bytes), max(1, max_slots) * self.pages_per_row + 1)
        if num_pages - 1 < self.pages_per_row:
            raise ValueError(f"KV budget holds {num_pages - 1} pages but one row of {max_seq_len} tokens needs {self.pages_per_row}")
        # Pages are handed out as rows grow, so the slot count is not tied to the worst-case length;
        # a row that cannot grow because the pool ran dry is preempted and generated again later.
        self.max_slots = max(b for b in (*self.BUCKETS, 4, 2, 1) if b <= max(1, min(max_slots, num_pages - 1)))
        self.pool = PagePool(num_pages)
        shape = (num_pages, self.n_kv, PAGE, cfg.head_dim)
        per = math.prod(shape)
        if kv_storage is None:
            kv_storage = torch.zeros(2 * cfg.n_layers * per, dtype=torch.bfloat16, device=self.dev)
        self.kcache = [kv_storage[(2 * l) * per:(2 * l + 1) * per].view(shape) for l in range(cfg.n_layers)]
        self.vcache = [kv_storage[(2 * l + 1) * per:(2 * l + 2) * per].view(shape) for l in range(cfg.n_layers)]
        n = self.max_slots
        i32 = dict(dtype=torch.int32, device=self.dev)
        self.group_rows = torch.full((n, self.GROUP_MAX), -1, **i32)
        self.group_shared = torch.zeros(n, **i32)
        self.row_key0 = torch.zeros(n, **i32)
        self._group_state = None
        self.token = torch.zeros(n, **i32)
        self.pos = torch.zeros(n, **i32)
        self.seq_len = torch.zeros(n, **i32)
        self.active = torch.zeros(n, **i32)
        self.gen_count = torch.zeros(n, **i32)
        self.forced_len = torch.zeros(n, **i32)
        self.forced = torch.full((n,), -1, **i32)
        self.slot_ids = torch.arange(n, **i32)
        self.page_table = torch.zeros((n, self.pages_per_row), **i32)
        self.sampled = torch.zeros(n, **i32)
        self.sampled_lp = torch.zeros(n, dtype=torch.float32, device=self.dev)
        self.n_finished = torch.zeros(1, **i32)
        self.step_counter = torch.zeros(1, dtype=torch.int64, device=self.dev)
        self.out_tok: Optional[torch.Tensor] = None
        self.out_lp: Optional[torch.Tensor] = None
        self._graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        self._graph_launches: Dict[tuple, int] = {}
        self.kv_bytes = 2 * cfg.n_layers * math.prod(shape) * 2

    # ------------------------------------------------------------------ decode step (graph body)
    def _nsplit(self, b: int) -> int:
        ctas = b * self.n_heads
        return 1 if ctas >= 296 else min(8, (296 + ctas - 1) // ctas)

    def _decode_body(self, b: int, temperature: float, greedy: bool, seed: int, top_k: int = 0, top_p: float = 1.0) -> None:
        m = self.model
        # chaining the step's kernels as programmatic dependents hides launch gaps at small batches (-3.7 % at 8 rows)
        # and costs a little once the kernels are long (+0.8 % at 128 rows and more)
        # (a tensor-parallel step is made of short kernels at every batch size: always chained)
        K.set_pdl(b <= self.PDL_MAX_BATCH or getattr(m, "tp", 1) > 1)
        groups = (self.group_rows[:b], self.group_shared[:b], self.row_key0[:b]) if (self.group_attention and b >= self.group_min_batch) else None
        K.set_group_tc(self.group_tc)
        xf = m.decode_step(self.token[:b], self.pos[:b], self.slot_ids[:b], self.seq_len[:b], self.page_table[:b],
                           self.kcache, self.vcache, nsplit=self._nsplit(b), groups=groups)
        logits = m.lm_logits(xf, decode=True)
        K.decode_prepare(self.active[:b], self.gen_count[:b], self.forced_len[:b], self.forced[:b], self.eos_id)
        K.sample(logits, temperature, greedy, seed, forced=self.forced[:b], token_out=self.sampled[:b],
                 logp_out=self.sampled_lp[:b], seed_offset=self.step_counter, top_k=top_k, top_p=top_p)
        K.decode_advance(self.sampled[:b], self.sampled_lp[:b], self.token[:b], self.pos[:b], self.seq_len[:b],
                         self.active[:b], self.gen_count[:b], self.out_tok[:b], self.out_lp[:b], self.eos_id,
                         self.n_finished, self.step_counter)
        K.set_pdl(True)

    def _step(self, b: int, temperature: float, greedy: bool, seed: int, top_k: int = 0, top_p: float = 1.0) -> None:
        if not self.use_graphs:
            self._decode_body(b, temperature, greedy, seed, top_k, top_p)
            return
        key = (b, self.out_tok.shape[1], float(temperature), bool(greedy), int(seed), self.out_tok.data_ptr(), int(top_k), float(top_p),
               self.group_attention)
        g = self._graphs.get(key)
        if g is None:
            # warm up and capture with every slot parked, so neither pass advances real rows
            saved = (self.active.clone(), self.n_finished.clone(), self.step_counter.clone())
            self.active.zero_()
            cur = torch.cuda.current_stream()
            side = torch.cuda.Stream(device=self.dev)
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                self._decode_body(b, temperature, greedy, seed, top_k, top_p)
            cur.wait_stream(side)
            g = torch.cuda.CUDAGraph()
            n0 = _lib.launch_count()
            with torch.cuda.graph(g):
                self._decode_body(b, temperature, greedy, seed, top_k, top_p)
            self._graph_launches[key] = _lib.launch_count() - n0
            _lib.add_launches(-self._graph_launches[key])  # capture itself executes nothing
            self.active.copy_(saved[0])
            self.n_finished.copy_(saved[1])
            self.step_counter.copy_(saved[2])
            self._graphs[key] = g
        g.replay()
        _lib.add_launches(self._graph_launches[key])

    # ------------------------------------------------------------------ prefill of admitted rows
    def _prefill(self, prompts: List[torch.Tensor], slots: List[int]) -> torch.Tensor:
        """Run the prompts through the model, store their K/V through the page-table rows of ``slots`` and return
        the logits at each prompt's last position ``[len(prompts), V]``."""
        cfg, dev = self.cfg, self.dev
        lens = [int(p.numel()) for p in prompts]
        tokens = torch.cat(prompts).to(device=dev, dtype=torch.int32)
        pos = torch.cat([torch.arange(l, dtype=torch.int32) for l in lens]).to(dev)
        seq_id = torch.cat([torch.full((l,), s, dtype=torch.int32) for l, s in zip(lens, slots)]).to(dev)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)

        k_col0, v_col0, n_kv = self.model.kv_columns()

        def sink(layer: int, qkv: torch.Tensor) -> None:
            K.kv_append(qkv, k_col0, v_col0, seq_id, pos, self.page_table, self.kcache[layer],
                        self.vcache[layer], n_kv, cfg.head_dim)

        xf, _ = self.model.forward(tokens, pos, cu, max(lens), keep=False, kv_sink=sink)
        last = (cu[1:] - 1).contiguous()
        return self.model.lm_logits(K.gather_rows(xf, last))

    def _start_rows(self, logits: torch.Tensor, lens: List[int], slots: List[int], forced: Optional[List[int]], temperature: float,
                    greedy: bool, seed: int, max_new: int, top_k: int = 0, top_p: float = 1.0) -> None:
        """Sample the first token of every admitted row from its prompt's last-position logits (one row of ``logits``
        per slot) and initialise the slot state for decoding."""
        dev = self.dev
        sl = torch.tensor(slots, dtype=torch.long, device=dev)
        lens_t = torch.tensor(lens, dtype=torch.int32, device=dev)
        f_len = torch.tensor(forced if forced is not None else [0] * len(slots), dtype=torch.int32, device=dev)
        first_forced = torch.where(f_len == 1, torch.full_like(f_len, self.eos_id), torch.full_like(f_len, -1))
        tok, lp = K.sample(logits, temperature, greedy, seed ^ 0x5DEECE66D, forced=first_forced, seed_offset=self.step_counter,
                           top_k=top_k, top_p=top_p)
        done = (tok == self.eos_id) | (max_new <= 1)
        self.out_tok[sl, 0] = tok
        self.out_lp[sl, 0] = lp
        self.gen_count[sl] = 1
        self.forced_len[sl] = f_len
        self.active[sl] = (~done).int()
        self.token[sl] = tok
        self.pos[sl] = lens_t
        self.seq_len[sl] = torch.where(done, torch.zeros_like(lens_t), lens_t + 1)
        self.n_finished += done.sum().int()

    # ------------------------------------------------------------------ public entry
    @torch.no_grad()
    def generate(self, prompts, max_new: int, *, temperature: float = 1.0, greedy: bool = False, seed: int = 0,
                 forced_lens=None, group_size: int = 1, top_k: int = 0, top_p: float = 1.0) -> GenerationResult:
        """Generate up to ``max_new`` tokens for every prompt (a ``[N, S]`` int tensor or a list of
        1-D tensors). ``forced_lens[i] > 0`` makes row ``i`` emit EOS as its ``forced_lens[i]``-th
        token (synthetic length control for benchmarks); natural EOS and the cap apply regardless.
        ``top_k`` / ``top_p`` restrict sampling (the recorded log-probs stay those of the full softmax).

        ``group_size = K`` declares that rows ``g*K .. g*K + K - 1`` carry the SAME prompt (K samples per prompt,
        GRPO): the prompt is prefilled once per group, its full KV pages are shared by the group's page-table
        rows (a reference count frees them with the last row), and the first token of every row is drawn from the
        one set of last-position logits. Rows of a group decode next to each other, so the shared pages are read
        from HBM about once per group and step instead of once per row."""
        dev = self.dev
        rows = [p for p in prompts] if not isinstance(prompts, torch.Tensor) else [prompts[i] for i in range(prompts.shape[0])]
        N = len(rows)
        G = max(1, int(group_size))
        if N % G:
            raise ValueError(f"{N} rows do not form groups of {G}")
        if G > 1 and isinstance(prompts, torch.Tensor):
            grouped = prompts.reshape(N // G, G, -1)
            if not bool((grouped == grouped[:, :1]).all()):
                raise ValueError(f"group_size={G}: the rows of a group must carry the same prompt")
        longest = max(int(r.numel()) for r in rows)
        if longest + max_new > self.max_seq_len:
            raise ValueError(f"prompt ({longest}) + max_new ({max_new}) exceeds max_seq_len ({self.max_seq_len})")
        forced = None if forced_lens is None else [int(x) for x in forced_lens]
        n = self.max_slots
        if self.out_tok is None or self.out_tok.shape[1] != max_new:  # kept across calls so captured graphs stay valid
            self.out_tok = torch.empty((n, max_new), dtype=torch.int32, device=dev)
            self.out_lp = torch.empty((n, max_new), dtype=torch.float32, device=dev)
            self._graphs.clear()
        self.out_tok.fill_(self.pad_id)
        self.out_lp.zero_()
        res_tok = torch.full((N, max_new), self.pad_id, dtype=torch.int32, device=dev)
        res_lp = torch.zeros((N, max_new), dtype=torch.float32, device=dev)
        res_len = torch.zeros(N, dtype=torch.int32, device=dev)
        for t in (self.active, self.seq_len, self.gen_count, self.n_finished, self.page_table, self.forced_len):
            t.zero_()
        self.pool = PagePool(self.pool.num_pages)      # a call that raised half way must not leak pages
        self._group_state = None
        self.group_shared.zero_()
        self.row_key0.zero_()
        slot_row = [-1] * n
        slot_pages: List[List[int]] = [[] for _ in range(n)]   # pages a slot owns (the shared prompt pages are not in here)
        slot_shared = [0] * n      # leading page-table entries that alias the group's shared prompt pages
        slot_bound = [0] * n       # upper bound on the tokens a slot holds (prompt + decode steps run since admission)
        slot_prompt = [0] * n
        queue = list(range(N))
        retired = 0
        counters = dict(prefill_calls=0, decode_steps=0, prefill_tokens=0, compactions=0, host_syncs=0, kv_pages_taken=0,
                        kv_pages_returned=0, kv_preemptions=0, live_slots_peak=0, graph_replays=0, shared_prompt_pages=0,
                        prompts_prefilled=0)
        seen_finished = 0
        horizon = self.sync_interval
        watermark = max(1, self.pool.num_pages // 20)     # pages kept free at admission so live rows can grow
        # per group of rows with one prompt: the shared full pages, the page that holds the prompt's ragged tail (rows copy
        # it into their own first page), the last-position logits, and how many of its rows have not retired yet
        groups: Dict[int, dict] = {}

        def pages_for(tokens: int) -> int:
            return min(self.pages_per_row, (tokens + PAGE - 1) // PAGE)

        def shared_pages_of(plen: int) -> int:
            return plen // PAGE if G > 1 else 0

        def release(slots_gone: List[int]) -> None:
            for s in slots_gone:
                counters["kv_pages_returned"] += len(slot_pages[s])
                self.pool.give(slot_pages[s])
                slot_pages[s] = []
                slot_row[s] = -1
                slot_shared[s] = 0

        def retire(slots_done: List[int]) -> None:
            nonlocal retired
            if not slots_done:
                return
            s_idx = torch.tensor(slots_done, dtype=torch.long, device=dev)
            r_idx = torch.tensor([slot_row[s] for s in slots_done], dtype=torch.long, device=dev)
            res_tok[r_idx] = self.out_tok[s_idx]
            res_lp[r_idx] = self.out_lp[s_idx]
            res_len[r_idx] = self.gen_count[s_idx]
            self.out_tok[s_idx] = self.pad_id
            self.out_lp[s_idx] = 0
            self.page_table[s_idx] = 0
            for s in slots_done:
                g = groups.get(slot_row[s] // G)
                if g is not None:
                    g["refs"] -= 1
                    if g["refs"] == 0:                   # last row of the group: the shared prompt pages go back
                        back = g["pages"] + ([g["tail"]] if g["tail"] else [])
                        counters["kv_pages_returned"] += len(back)
                        self.pool.give(back)
                        del groups[slot_row[s] // G]
            release(slots_done)
            retired += len(slots_done)

        def preempt(victims: List[int]) -> None:
            """Give a row's own pages back and queue it again from its prompt (its partial output is dropped; the
            group's shared prompt pages stay, the row is still owed)."""
            s_idx = torch.tensor(victims, dtype=torch.long, device=dev)
            for arr in (self.active, self.seq_len, self.gen_count, self.forced_len, self.page_table, self.out_lp):
                arr[s_idx] = 0
            self.out_tok[s_idx] = self.pad_id
            for s in victims:
                queue.insert(0, slot_row[s])
            release(victims)
            counters["kv_preemptions"] += len(victims)

        def grow(live: List[int]) -> List[int]:
            """Extend every live row's page list to cover the next ``horizon`` decode steps; preempts
            the rows with the least progress when the pool cannot cover it. Returns the rows still live."""
            live = list(live)
            while True:
                want = {s: pages_for(slot_bound[s] + horizon) - slot_shared[s] - len(slot_pages[s]) for s in live}
                total = sum(v for v in want.values() if v > 0)
                if total <= self.pool.available() or len(live) <= 1:
                    break
                victim = min(live, key=lambda s: (slot_bound[s] - slot_prompt[s], -s))
                preempt([victim])
                live.remove(victim)
            idx, val = [], []
            for s in live:
                k = want[s]
                if k > 0:
                    have = slot_shared[s] + len(slot_pages[s])
                    new = self.pool.take(k)
                    counters["kv_pages_taken"] += k
                    slot_pages[s].extend(new)
                    idx.extend(s * self.pages_per_row + have + j for j in range(k))
                    val.extend(new)
            if idx:
                self.page_table.view(-1).index_copy_(0, torch.tensor(idx, dtype=torch.long, device=dev),
                                                     torch.tensor(val, dtype=torch.int32, device=dev))
            return live

        def copy_page(src: int, dst: List[int]) -> None:
            """Copy one KV page (all layers, K and V) onto the pages ``dst``."""
            per = self.kcache[0].numel()
            flat = self.kcache[0].new_empty(0).set_(self.kcache[0].untyped_storage(), self.kcache[0].storage_offset(),
                                                    (2 * self.cfg.n_layers, self.kcache[0].shape[0], per // self.kcache[0].shape[0]))
            d = torch.tensor(dst, dtype=torch.long, device=dev)
            flat[:, d] = flat[:, src].unsqueeze(1)

        while retired < N:
            free = [s for s in range(n) if slot_row[s] < 0]
            # admit in batches: a prefill call stalls decoding, so wait until several slots are free
            if queue and len(free) >= min(len(queue), max(1, n // 8)):
                new_rows, new_slots = [], []
                budget = self.pool.available() - (watermark if any(r >= 0 for r in slot_row) else 0)
                opening = set()                                  # groups whose prompt this admission prefills
                for s in free:
                    if not queue:
                        break
                    r = queue[0]
                    plen = int(rows[r].numel())
                    sh = shared_pages_of(plen)
                    need = pages_for(plen + 1 + horizon) - sh
                    g = r // G
                    if sh and g not in groups and g not in opening:
                        need += sh + (1 if plen % PAGE else 0)   # the group's shared pages (+ its tail page) come with its first row
                    if need > budget:
                        break
                    budget -= need
                    if sh:
                        opening.add(g)
                    new_rows.append(queue.pop(0))
                    new_slots.append(s)
                if new_rows:
                    table = torch.zeros((len(new_rows), self.pages_per_row), dtype=torch.int32)
                    prefill_rows, prefill_slots = [], []
                    for j, (r, s) in enumerate(zip(new_rows, new_slots)):
                        plen = int(rows[r].numel())
                        sh = shared_pages_of(plen)
                        g = r // G
                        if sh and g not in groups:
                            shared = self.pool.take(sh)
                            tail = self.pool.take(1)[0] if plen % PAGE else 0
                            counters["kv_pages_taken"] += sh + (1 if tail else 0)
                            counters["shared_prompt_pages"] += sh
                            groups[g] = dict(pages=shared, tail=tail, refs=G, logits=None, plen=plen)
                            prefill_rows.append(r)
                            prefill_slots.append(s)
                        elif not sh:
                            prefill_rows.append(r)
                            prefill_slots.append(s)
                        own = self.pool.take(pages_for(plen + 1 + horizon) - sh)
                        counters["kv_pages_taken"] += len(own)
                        slot_pages[s], slot_row[s], slot_prompt[s], slot_bound[s], slot_shared[s] = own, r, plen, plen + 1, sh
                        if sh:
                            table[j, :sh] = torch.tensor(groups[g]["pages"], dtype=torch.int32)
                        table[j, sh:sh + len(own)] = torch.tensor(own, dtype=torch.int32)
                    self.page_table[torch.tensor(new_slots, dtype=torch.long, device=dev)] = table.to(dev)
                    if prefill_rows:
                        logits = self._prefill([rows[r] for r in prefill_rows], prefill_slots)
                        counters["prefill_calls"] += 1
                        counters["prompts_prefilled"] += len(prefill_rows)
                        counters["prefill_tokens"] += sum(int(rows[r].numel()) for r in prefill_rows)
                    if G > 1:
                        for j, (r, s) in enumerate(zip(prefill_rows, prefill_slots)):
                            g = groups.get(r // G)
                            if g is not None and g["logits"] is None:
                                g["logits"] = logits[j].clone()
                                if g["tail"]:               # keep the prompt's ragged tail for the rows that come later
                                    copy_page(slot_pages[s][0], [g["tail"]])
                        for r, s in zip(new_rows, new_slots):   # rows that alias an already prefilled prompt need its tail
                            g = groups.get(r // G)
                            if g is not None and g["tail"] and not (r in prefill_rows):
                                copy_page(g["tail"], [slot_pages[s][0]])
                        row_logits = torch.stack([groups[r // G]["logits"] if (r // G) in groups else logits[prefill_rows.index(r)]
                                                  for r in new_rows])
                    else:
                        row_logits = logits
                    self._start_rows(row_logits, [int(rows[r].numel()) for r in new_rows], new_slots,
                                     None if forced is None else [forced[r] for r in new_rows], temperature, greedy, seed, max_new,
                                     top_k, top_p)
            live = [s for s in range(n) if slot_row[s] >= 0]
            if not live:
                if queue:
                    raise RuntimeError("KV page pool cannot hold a single prompt; raise the KV budget")
                break
            used = max(live) + 1
            if not queue and len(live) <= self._bucket(used) // 2 and self._bucket(len(live)) < self._bucket(used):
                self._compact(live, slot_row, slot_pages, slot_bound, slot_prompt, slot_shared)
                counters["compactions"] += 1
                live = list(range(len(live)))
            live = grow(live)
            used = max(live) + 1
            counters["live_slots_peak"] = max(counters["live_slots_peak"], len(live))
            b = self._bucket(used)
            if self.group_attention:
                self._sync_groups(live, slot_row, slot_shared, G)
            for _ in range(horizon):
                self._step(b, temperature, greedy, seed, top_k, top_p)
            counters["decode_steps"] += horizon
            counters["graph_replays"] += horizon if self.use_graphs else 0
            for s in live:
                slot_bound[s] = min(slot_bound[s] + horizon, slot_prompt[s] + max_new)
            nf = int(self.n_finished.item())
            counters["host_syncs"] += 1
            if self.check_status_every_sync:
                K.check_status()
            if nf != seen_finished:
                seen_finished = nf
                act = self.active.tolist()
                retire([s for s in range(n) if slot_row[s] >= 0 and not act[s]])
        counters["kv_bytes"] = float(self.kv_bytes)
        return GenerationResult(res_tok, res_lp, res_len, counters)

    def _sync_groups(self, live: List[int], slot_row: List[int], slot_shared: List[int], G: int) -> None:
        """Tell the attention kernel which live slots share prompt pages: members of a prompt group (at least
        ``GROUP_MIN`` of them live, at most ``GROUP_MAX`` per kernel group) and the number of shared keys."""
        by_prompt: Dict[int, List[int]] = {}
        for s in live:
            if slot_shared[s] > 0:
                by_prompt.setdefault(slot_row[s] // G, []).append(s)
        rows, shared, key0 = [], [], {}
        for g in sorted(by_prompt):
            members = sorted(by_prompt[g])
            for i in range(0, len(members), self.GROUP_MAX):
                chunk = members[i:i + self.GROUP_MAX]
                if len(chunk) < self.GROUP_MIN:
                    continue
                rows.append(chunk + [-1] * (self.GROUP_MAX - len(chunk)))
                shared.append(slot_shared[chunk[0]] * PAGE)
                for s in chunk:
                    key0[s] = shared[-1]
        state = (tuple(map(tuple, rows)), tuple(shared))
        if state == self._group_state:
            return
        self._group_state = state
        n = self.max_slots
        gr = torch.full((n, self.GROUP_MAX), -1, dtype=torch.int32)
        gs = torch.zeros(n, dtype=torch.int32)
        k0 = torch.zeros(n, dtype=torch.int32)
        if rows:
            gr[: len(rows)] = torch.tensor(rows, dtype=torch.int32)
            gs[: len(shared)] = torch.tensor(shared, dtype=torch.int32)
            for s, v in key0.items():
                k0[s] = v
        self.group_rows.copy_(gr.to(self.dev))
        self.group_shared.copy_(gs.to(self.dev))
        self.row_key0.copy_(k0.to(self.dev))

    def _bucket(self, used: int) -> int:
        for b in sorted((*self.BUCKETS, 4, 2, 1)):
            if b >= used and b <= self.max_slots:
                return b
        return self.max_slots

    def _compact(self, live: List[int], slot_row: List[int], slot_pages: List[List[int]], slot_bound: List[int],
                 slot_prompt: List[int], slot_shared: List[int]) -> None:
        """Move live slots to the front (state and page-table rows only; KV pages stay where they are)."""
        k = len(live)
        idx = torch.tensor(live, dtype=torch.long, device=self.dev)
        for arr in (self.token, self.pos, self.seq_len, self.active, self.gen_count, self.forced_len, self.page_table,
                    self.out_tok, self.out_lp):
            moved = arr[idx].clone()
            arr[:k] = moved
            if arr is self.out_tok:
                arr[k:] = self.pad_id
            elif arr is not self.pos and arr is not self.token:
                arr[k:] = 0
        rows = [slot_row[s] for s in live]
        pages = [slot_pages[s] for s in live]
        bounds = [slot_bound[s] for s in live]
        prompts = [slot_prompt[s] for s in live]
        shared = [slot_shared[s] for s in live]
        for s in range(len(slot_row)):
            slot_shared[s] = shared[s] if s < k else 0
            slot_row[s] = rows[s] if s < k else -1
            slot_pages[s] = pages[s] if s < k else []
            slot_bound[s] = bounds[s] if s < k else 0
            slot_prompt[s] = prompts[s] if s < k else 0
