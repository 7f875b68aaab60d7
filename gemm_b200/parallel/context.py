"""Context parallelism: the KV positions of every sequence are sharded block-cyclically over the ranks.

Rank r stores the K/V of the position blocks b with ``b % world == r`` (block = 128 positions) in its own paged cache; every
rank holds the same queries, runs the flash kernel over its local shard only and gets partials (O normalised by its own
sum, base-2 log-sum-exp); the partials are exchanged with peer stores into every rank's heap and merged with the rule of
the split-KV decode, so all ranks end with identical outputs.  This is the reference's scheme for its long-context decode
(a64fx/m3/m3_ep_runner.c:121-140, common/glm5.h:285-298: all-reduce-MAX of the per-head maxima followed by an
all-reduce-SUM of the rescaled [sumexp | out]); here the two all-reduces are one all-gather of ``Hq * (D + 1)`` floats per
token and rank plus the merge kernel.  As in the reference, tensor-parallel attention is off under context parallelism.

Given to ``Engine`` as its ``par`` (block = the engine's page size) the same object runs whole models: weights are replicated,
page g of a sequence lives on rank ``g % world`` as that rank's page ``g // world``, so the cache of a rank holds 1 / world of
every sequence.  A decode step runs the token-wise layers replicated and the attention as above.  A prefill is sequence
parallel: every rank runs the layers over the tokens of its own pages only (1 / world of the GEMM work; pages are dealt round
robin, so the causal attention work is balanced too), writes their K / V into its cache, and per layer the ranks all-gather the
K / V rows of the prompt into a staging buffer that the flash kernel reads through a block table (one attention item per owned
page: its 128 queries against the pages ``0 .. g``).  The reference has no prefill of its own under context parallelism (it
feeds the prompt through the decode function token by token, common/m3_impl.h:643-683).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..models.transformer import ForwardBatch, SingleProcess
from ..ops import attention as att
from .fabric import Fabric


def merge_two(o1: torch.Tensor, l1: torch.Tensor, o2: torch.Tensor, l2: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Merge of two attention partials (outputs normalised by their own sums, base-2 log-sum-exps); symmetric in its arguments,
    so two ranks that swap partials compute the same bits."""
    m = torch.maximum(l1, l2)
    safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w1, w2 = torch.exp2(l1 - safe), torch.exp2(l2 - safe)
    den = w1 + w2
    o = (w1[..., None] * o1 + w2[..., None] * o2) / den.clamp_min(1e-30)[..., None]
    return o, safe + torch.log2(den)


def _swap(send: torch.Tensor, dst: int, src: int, group) -> torch.Tensor:
    recv = torch.empty_like(send)
    ops = [dist.P2POp(dist.isend, send, dist.get_global_rank(group, dst) if group is not None else dst, group),
           dist.P2POp(dist.irecv, recv, dist.get_global_rank(group, src) if group is not None else src, group)]
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    return recv


def merge_ring(o: torch.Tensor, lse: torch.Tensor, group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """The partials of all ranks merged by passing them around the ring: ``world - 1`` hops, each rank forwards what it received
    last and folds it into its running result.  Every rank ends with the merge of all partials, folded in a different order, so
    the results agree to rounding only: a benchmark variant (the reference times the same pattern,
    a64fx/utofu-tests/ring_attn_bench.c:19-27), not what the engine runs."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    pay = torch.cat([o.float().reshape(-1, o.shape[-1]), lse.float().reshape(-1, 1)], dim=1).contiguous()
    acc_o, acc_l, cur = o.float(), lse.float(), pay
    for _ in range(world - 1):
        cur = _swap(cur, (rank + 1) % world, (rank - 1) % world, group)
        acc_o, acc_l = merge_two(acc_o, acc_l, cur[:, :-1].reshape(o.shape), cur[:, -1].reshape(lse.shape))
    return acc_o, acc_l


def merge_tree(o: torch.Tensor, lse: torch.Tensor, group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """The same by recursive doubling: ``log2(world)`` rounds, in round k rank r swaps its running result with rank ``r ^ 2^k``.
    Both partners compute the same merge, so all ranks end with identical bits.  A world size that is not a power of two folds
    its upper ranks into the lower ones first and hands them the result at the end (the reference measures this against the ring,
    a64fx/utofu-tests/ring_attn_bench.c:23-27)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    pof2 = 1 << (world.bit_length() - 1)
    acc_o, acc_l = o.float(), lse.float()
    pack = lambda a, b: torch.cat([a.reshape(-1, a.shape[-1]), b.reshape(-1, 1)], dim=1).contiguous()

    def send(t, dst):
        dist.send(t, dist.get_global_rank(group, dst) if group is not None else dst, group=group)

    def recv(like, src):
        buf = torch.empty_like(like)
        dist.recv(buf, dist.get_global_rank(group, src) if group is not None else src, group=group)
        return buf
    if rank >= pof2:                                             # an upper rank: give, then wait for the result
        send(pack(acc_o, acc_l), rank - pof2)
        res = recv(pack(acc_o, acc_l), rank - pof2)
        return res[:, :-1].reshape(o.shape), res[:, -1].reshape(lse.shape)
    if rank + pof2 < world:
        got = recv(pack(acc_o, acc_l), rank + pof2)
        acc_o, acc_l = merge_two(acc_o, acc_l, got[:, :-1].reshape(o.shape), got[:, -1].reshape(lse.shape))
    k = 1
    while k < pof2:
        peer = rank ^ k
        got = _swap(pack(acc_o, acc_l), peer, peer, group)
        acc_o, acc_l = merge_two(acc_o, acc_l, got[:, :-1].reshape(o.shape), got[:, -1].reshape(lse.shape))
        k <<= 1
    if rank + pof2 < world:
        send(pack(acc_o, acc_l), rank + pof2)
    return acc_o, acc_l


class ContextParallel(SingleProcess):
    def __init__(self, group, device: torch.device, block: int = 128, fused: bool = True, max_tokens: int = 256, hq: int = 32,
                 head_dim: int = 128, max_splits: int = 1):
        self.group, self.device, self.block = group, device, block
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.cp_world, self.cp_rank = self.world, self.rank
        self._stage = {}
        self.fused = fused and device.type == "cuda"
        self.max_tokens, self.hq, self.d, self.max_splits = max_tokens, hq, head_dim, max_splits
        self.fab: Optional[Fabric] = None
        if self.fused:
            per = max_splits * max_tokens * hq * (head_dim + 1) * 4
            self.fab = Fabric(group, device, self.world * per + (1 << 20))
            self.ag = self.fab.make_exchange(per, chunks=8)

    # ------------------------------------------------------------------------------------------ layout
    def owner(self, pos: int) -> int:
        return (pos // self.block) % self.world

    def local_index(self, pos: int) -> int:
        """Index of global position ``pos`` inside its owner's shard."""
        return (pos // (self.block * self.world)) * self.block + pos % self.block

    def local_len(self, kv_len: int, rank: Optional[int] = None) -> int:
        """How many of the positions ``[0, kv_len)`` the rank owns."""
        r = self.rank if rank is None else rank
        full, rem = divmod(kv_len, self.block * self.world)
        return full * self.block + min(max(rem - r * self.block, 0), self.block)

    def local_pages(self, n_pages: int, rank: Optional[int] = None) -> int:
        """How many of the pages ``[0, n_pages)`` of a sequence the rank stores."""
        r = self.rank if rank is None else rank
        return (n_pages - r + self.world - 1) // self.world if n_pages > r else 0

    def shard_positions(self, kv_len: int, rank: Optional[int] = None) -> Sequence[int]:
        r = self.rank if rank is None else rank
        return [p for p in range(kv_len) if self.owner(p) == r]

    # ------------------------------------------------------------------------------------------ attention
    def attention(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cu_q: torch.Tensor, local_kv_len: torch.Tensor,
                  block_table: torch.Tensor, page_size: int, work: torch.Tensor, num_splits: int = 1, decode: bool = False) -> torch.Tensor:
        """``q`` bf16 [T, Hq, D] (the same on every rank, pre-scaled as the flash kernel expects; one decode token per sequence);
        caches, ``local_kv_len`` and ``block_table`` describe THIS rank's shard.  ``num_splits`` (<= ``max_splits``; ``work`` built
        for it): the rank's shard is cut into that many KV ranges, each a partial of its own in the merge.  ``decode`` selects the
        decode-specialised kernel.  Returns bf16 [T, Hq, D], identical on all ranks."""
        t, hq, d = q.shape
        ns = num_splits
        po, pl = att.attention_partial(q, k_cache, v_cache, cu_q, local_kv_len, block_table, page_size, work, num_splits=ns, causal=False,
                                       decode=decode)
        mine = torch.cat([po.reshape(ns * t, hq * d), pl.reshape(ns * t, hq)], dim=1).contiguous()      # [S * T, Hq * (D + 1)] f32
        if self.fused:
            assert t <= self.max_tokens and ns <= self.max_splits and hq == self.hq and d == self.d
            rows = self.max_splits * self.max_tokens
            buf = torch.zeros(rows, hq * (d + 1), dtype=torch.float32, device=q.device)
            buf[: ns * t] = mine
            allp = self.ag.all_gather(buf).view(torch.float32).view(self.world, rows, hq * (d + 1))[:, : ns * t]
        else:
            parts = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(parts, mine, group=self.group)
            allp = torch.stack(parts)
        part_o = allp[:, :, : hq * d].reshape(self.world * ns, t * hq, d).contiguous()
        part_lse = allp[:, :, hq * d:].reshape(self.world * ns, t * hq).contiguous()
        out, _ = att.combine_partials(part_o, part_lse)
        return out.reshape(t, hq, d)

    # ------------------------------------------------------------------------------------------ whole-model prefill
    def build_prefill(self, prompts: Sequence[torch.Tensor], local_pages: Sequence[Sequence[int]], hq: int, hkv: int, device,
                      seq_slots: Optional[Sequence[int]] = None) -> Tuple[ForwardBatch, List[int]]:
        """The forward batch of THIS rank for a prefill of whole prompts (every sequence from position 0), and the sequences
        whose last token the rank holds (their logits are the first ``len(owned)`` rows of the forward's output).
        ``local_pages[s]``: the rank's cache pages of sequence ``s`` in order (its page ``i`` is the sequence's page
        ``rank + i * world``).  Attention items are the rank's pages; their block tables address the gathered staging buffer,
        where rank q's region (``p_local`` pages) holds its pages of sequence 0, then of sequence 1, and so on."""
        page, w, r = self.block, self.world, self.rank
        b = len(prompts)
        lens = [int(p.numel()) for p in prompts]
        gp = [(n + page - 1) // page for n in lens]
        first = [[0] * (b + 1) for _ in range(w)]
        for q in range(w):
            for s in range(b):
                first[q][s + 1] = first[q][s] + self.local_pages(gp[s], q)
        p_local = max(max(first[q][b] for q in range(w)), 1)
        ids, pos, slots, cu, kvl, tables, rows, owned = [], [], [], [0], [], [], [], []
        send = [0] * (p_local * page)
        for s in range(b):
            for g in range(r, gp[s], w):
                lo, hi = g * page, min((g + 1) * page, lens[s])
                cache_page = int(local_pages[s][g // w])
                ids.append(prompts[s][lo:hi].to(torch.int32).cpu())
                pos.extend(range(lo, hi))
                slots.extend(cache_page * page + i for i in range(hi - lo))
                st = (first[r][s] + g // w) * page
                send[st: st + hi - lo] = [cache_page * page + i for i in range(hi - lo)]
                cu.append(cu[-1] + hi - lo)
                kvl.append(hi)
                tables.append([(g2 % w) * p_local + first[g2 % w][s] + g2 // w for g2 in range(g + 1)])
                if hi == lens[s]:
                    rows.append(cu[-1] - 1)
                    owned.append(s)
        if not pos:
            # a rank without a page of any prompt still joins every layer's collectives: it runs one token that stores nothing
            ids, pos, slots, cu, kvl, tables = [torch.zeros(1, dtype=torch.int32)], [0], [-1], [0, 1], [1], [[0]]
        if not rows:
            rows = [0]
        i32 = dict(dtype=torch.int32, device=device)
        q_lens = [cu[i + 1] - cu[i] for i in range(len(cu) - 1)]
        bt = torch.zeros(len(tables), max(len(t) for t in tables), dtype=torch.int32)
        for i, t in enumerate(tables):
            bt[i, : len(t)] = torch.tensor(t, dtype=torch.int32)
        fb = ForwardBatch(ids=torch.cat(ids).to(device), positions=torch.tensor(pos, **i32), slots=torch.tensor(slots, **i32),
                          cu_q=torch.tensor(cu, **i32), kv_len=torch.tensor(kvl, **i32), block_table=bt.to(device),
                          work=att.build_work(q_lens, hq, hkv, 1).to(device), logit_rows=torch.tensor(rows, dtype=torch.int64, device=device),
                          num_splits=1, n_tokens=len(pos),
                          seq_slots=torch.tensor(list(seq_slots) if seq_slots is not None else list(range(b)), **i32), is_decode=False)
        fb.cp_send_slots = torch.tensor(send, dtype=torch.int64, device=device)
        return fb, owned

    def gather_kv(self, k_cache: torch.Tensor, v_cache: torch.Tensor, send_slots: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """All-gather of the prompt's K / V rows of one layer: every rank contributes the rows of ``send_slots`` of its cache
        (the staging order of ``build_prefill``); returns ``[world * len(send_slots), Hkv, D]`` caches for the flash kernel.
        The staging buffers are kept and reused by the next layer."""
        n = send_slots.numel()
        key = (n, k_cache.shape[1], k_cache.shape[2], k_cache.dtype, k_cache.device)
        if key not in self._stage:
            self._stage.clear()
            self._stage[key] = tuple(torch.empty(self.world * n, k_cache.shape[1], k_cache.shape[2], dtype=k_cache.dtype, device=k_cache.device)
                                     for _ in range(2))
        kg, vg = self._stage[key]
        for full, cache in ((kg, k_cache), (vg, v_cache)):
            mine = full[self.rank * n: (self.rank + 1) * n]
            torch.index_select(cache, 0, send_slots, out=mine)
            dist.all_gather([full[q * n: (q + 1) * n] for q in range(self.world)], mine, group=self.group)
        return kg, vg

    def merge_logits(self, logits: torch.Tensor, owned: Sequence[int], n_seqs: int) -> torch.Tensor:
        """Every rank's last-token logits (rows of the sequences it ``owned``) put together: ``f32 [n_seqs, V]`` on all ranks."""
        full = torch.zeros(n_seqs, logits.shape[1], dtype=torch.float32, device=logits.device)
        if owned:
            full[torch.tensor(list(owned), dtype=torch.int64, device=logits.device)] = logits[: len(owned)].float()
        dist.all_reduce(full, group=self.group)
        return full

    def close(self) -> None:
        if self.fab is not None:
            self.fab.close()
