"""Model executor for the continuous-batching scheduler: a Llama-style decoder running on the paged
KV cache with the native kernels (GEMM with fused SwiGLU / residual epilogues, RMSNorm, RoPE,
KV-cache write, FlashAttention-style prefill, paged decode, greedy sampling).

``execute_batch`` is the ``IModelExecutor.ExecuteBatchAsync`` of the reference
(src/MLFramework/Inference/ContinuousBatching/IModelExecutor.cs:8-16). Its attention path is what
``PagedAttentionLayer.ComputeAttention`` describes (src/MLFramework/Inference/PagedAttention/Layers/
PagedAttentionLayer.cs:102-144: project, update the KV cache block by block, attend over the
sequence's blocks, output projection) with the parts the reference stubs out (copy into blocks,
gather from blocks, the CUDA kernel) implemented.

Tensor parallel serving: every rank holds ``n_heads / W`` query heads, ``n_kv_heads / W`` KV heads and
``d_ff / W`` FFN columns; the partial outputs of the o- and down-projections are summed over ranks
by the one-shot in-kernel all-reduce over peer memory (latency bound: 2 MiB per layer at batch 256)
or a process-group all-reduce. Rank 0 runs the scheduler and broadcasts each iteration's plan.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from ..models.llama import Llama, LlamaConfig
from ..ops import native, reference
from ..ops.gemm import gemm
from .. import _lib
from .kv_cache import KVCacheBlockManager
from .scheduler import Batch, BatchOutput, Request


@dataclass
class ExecutorConfig:
    max_batch: int = 256
    max_seq_len: int = 4096
    prefill_chunk: int = 2048
    decode_split_tokens: int = 0          # 0: chosen from the batch size
    max_prefill_tokens: int = 8192        # first chunks of equal length are prefilled together up to this many tokens
    use_cuda_graphs: bool = True       # decode steps replay a captured graph per (batch bucket, length bucket)
    graph_warmup_steps: int = 2
    torch_ops: bool = False            # comparison arm: same scheduler and block tables, every operator from torch (cuBLAS
                                       # linears, F.rms_norm, SDPA over pages gathered by indexing), eager, NCCL reductions


class PagedLlamaExecutor:
    def __init__(self, model: Llama, kv: KVCacheBlockManager, config: Optional[ExecutorConfig] = None, tp=None):
        self.m, self.kv, self.cfg, self.tp = model, kv, config or ExecutorConfig(), tp
        self.mc: LlamaConfig = model.cfg
        p = next(model.parameters())
        self.device, self.dtype = p.device, p.dtype
        self.native = p.is_cuda and p.dtype == torch.bfloat16 and self.mc.head_dim == 128 and not self.cfg.torch_ops
        W = tp.world if tp is not None else 1
        self.hq, self.hkv = self.mc.n_heads // W, self.mc.n_kv_heads // W
        self.max_blocks = (self.cfg.max_seq_len + kv.block_size - 1) // kv.block_size
        self.tokens_generated = 0
        self._graphs = None
        self._ar_calls = 0
        if self.native and self.cfg.use_cuda_graphs and (tp is None or tp.world == 1 or tp.fused):
            from ..hal.cuda_graphs import CaptureOptions, CUDAGraphManager
            self._graphs = CUDAGraphManager(CaptureOptions(warmup_iterations=self.cfg.graph_warmup_steps))

    # ---- tensor-parallel reduction of partial projections
    def _ar_staging(self, T: int):
        """[T, d_model] view of one of two alternating peer-visible staging buffers for a row-parallel product.
        Two per transformer block, so a step (eager or a replayed graph) always starts on the same one."""
        tp = self.tp
        nbytes = max(self.cfg.max_batch, self.cfg.prefill_chunk, self.cfg.max_prefill_tokens) * self.mc.d_model * 2
        nbytes = (nbytes + 255) // 256 * 256
        buf = tp.symm_buffer("serve.ar2", 2 * nbytes)
        off = (self._ar_calls % 2) * nbytes
        self._ar_calls += 1
        return buf, off, buf.view(torch.bfloat16, T * self.mc.d_model, off).view(T, self.mc.d_model)

    def _row_parallel(self, a: torch.Tensor, w: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        """residual + sum over ranks of a @ w^T: the product lands in the staging buffer, one kernel
        synchronises with the peers and adds their partial sums."""
        T = a.shape[0]
        buf, off, stage = self._ar_staging(T)
        gemm(a, w, out=stage)
        out = torch.empty_like(residual)
        self.tp.symm.all_reduce_one_shot_sync(buf, out, T * self.mc.d_model, residual=residual, offset_bytes=off)
        return out

    def _reduce(self, partial: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        if self.tp is None or self.tp.world == 1:
            return partial + residual if residual is not None else partial
        tp = self.tp
        if tp.fused and partial.is_cuda:
            n = partial.numel()
            buf = tp.symm_buffer("serve.ar", self.cfg.max_batch * max(self.cfg.prefill_chunk, 1) * self.mc.d_model * 2
                                 if n * 2 > (1 << 22) else (1 << 22))
            buf.view(partial.dtype, n).copy_(partial.reshape(-1))
            tp.symm.barrier()
            out = torch.empty_like(partial)
            tp.symm.all_reduce_one_shot(buf, out, n, residual=residual)
            tp.symm.barrier()
            return out
        from ..dist.process_group import ReduceOp
        tp.pg.all_reduce(partial, ReduceOp.SUM)
        return partial + residual if residual is not None else partial

    # ---- one transformer block over T tokens
    def _block(self, li: int, blk, x: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, attend):
        mc = self.mc
        D = mc.head_dim
        attn = blk.attn if hasattr(blk, "attn") else None
        qkv_w = attn.qkv.weight if attn is not None else blk.qkv.weight
        o_w = attn.proj.weight if attn is not None else blk.o.weight
        gu_w = blk.mlp.gate_up.weight if hasattr(blk, "mlp") else blk.gate_up.weight
        dn_w = blk.mlp.down.weight if hasattr(blk, "mlp") else blk.down.weight
        cache = self.kv.caches[li]
        T = x.shape[0]
        if self.native:
            h, _, _ = native.norm_fwd(x, blk.norm1.weight, None, mc.norm_eps, True, want_stats=False)
            qkv = gemm(h, qkv_w)
            q = qkv[:, :self.hq * D].view(T, self.hq, D)
            k = qkv[:, self.hq * D:(self.hq + self.hkv) * D].view(T, self.hkv, D)
            v = qkv[:, (self.hq + self.hkv) * D:].view(T, self.hkv, D)
            native.rope_kv_write_(qkv, positions, slots, cache, self.hq, self.hkv, mc.rope_theta)
            a = attend(li, q, k, v)
            multi = self.tp is not None and self.tp.world > 1
            # A decode step (few rows, whole weights) streams weights: plain products let the GEMM split K over
            # all SMs, the residual stream takes the product as an accumulation, SwiGLU runs as its own pass.
            few_rows = T <= 256
            sync_ar = multi and self.tp.fused
            if sync_ar:
                x = self._row_parallel(a.reshape(T, self.hq * D), o_w, x)
            elif multi:
                x = self._reduce(gemm(a.reshape(T, self.hq * D), o_w), x)
            elif few_rows:
                gemm(a.reshape(T, self.hq * D), o_w, out=x, flags=_lib.EPI_ACCUM)
            else:
                x = gemm(a.reshape(T, self.hq * D), o_w, aux_in=x, flags=_lib.EPI_RESIDUAL)
            h, _, _ = native.norm_fwd(x, blk.norm2.weight, None, mc.norm_eps, True, want_stats=False)
            hid = native.swiglu_fwd(gemm(h, gu_w), interleaved=True) if few_rows else gemm(h, gu_w, flags=_lib.EPI_SWIGLU)
            if sync_ar:
                return self._row_parallel(hid, dn_w, x)
            if multi:
                return self._reduce(gemm(hid, dn_w), x)
            if few_rows:
                return gemm(hid, dn_w, out=x, flags=_lib.EPI_ACCUM)
            return gemm(hid, dn_w, aux_in=x, flags=_lib.EPI_RESIDUAL)
        if self.cfg.torch_ops:
            return self._block_torch(x, blk, qkv_w, o_w, gu_w, dn_w, cache, positions, slots, attend, li)
        # ---- PyTorch statement of the same block (CPU / fp32)
        h, _ = reference.rms_norm_ref(x, blk.norm1.weight, mc.norm_eps)
        qkv = F.linear(h.to(x.dtype), qkv_w)
        q = qkv[:, :self.hq * D].reshape(T, self.hq, D)
        k = qkv[:, self.hq * D:(self.hq + self.hkv) * D].reshape(T, self.hkv, D)
        v = qkv[:, (self.hq + self.hkv) * D:].reshape(T, self.hkv, D)
        q = reference.rope_ref(q, positions, mc.rope_theta).to(x.dtype)
        k = reference.rope_ref(k, positions, mc.rope_theta).to(x.dtype)
        flat = cache.view(-1, 2, self.kv.block_size, self.hkv, D)
        ok = slots >= 0
        blk_i, off = slots[ok] // self.kv.block_size, slots[ok] % self.kv.block_size
        flat[blk_i, 0, off] = k[ok]
        flat[blk_i, 1, off] = v[ok]
        a = attend(li, q, k, v)
        x = self._reduce(F.linear(a.reshape(T, self.hq * D).to(x.dtype), o_w), x)
        h, _ = reference.rms_norm_ref(x, blk.norm2.weight, mc.norm_eps)
        gu = F.linear(h.to(x.dtype), gu_w)
        hid = (F.silu(gu[:, 0::2].float()) * gu[:, 1::2].float()).to(x.dtype)
        return self._reduce(F.linear(hid, dn_w), x)

    def _block_torch(self, x, blk, qkv_w, o_w, gu_w, dn_w, cache, positions, slots, attend, li):
        """The block from torch operators in the model's dtype (the comparison arm on a GPU)."""
        mc, D, T = self.mc, self.mc.head_dim, x.shape[0]
        qkv = F.linear(F.rms_norm(x, (x.shape[-1],), blk.norm1.weight, mc.norm_eps), qkv_w)
        q = qkv[:, :self.hq * D].reshape(T, self.hq, D)
        k = qkv[:, self.hq * D:(self.hq + self.hkv) * D].reshape(T, self.hkv, D)
        v = qkv[:, (self.hq + self.hkv) * D:].reshape(T, self.hkv, D)
        inv = mc.rope_theta ** (-torch.arange(0, D, 2, device=x.device, dtype=torch.float32) / D)
        ang = positions.float()[:, None] * inv[None, :]
        c, sn = ang.cos()[:, None, :], ang.sin()[:, None, :]

        def rope(t):
            a, b = t[..., 0::2].float(), t[..., 1::2].float()
            return torch.stack((a * c - b * sn, a * sn + b * c), -1).flatten(-2).to(t.dtype)
        q, k = rope(q), rope(k)
        flat = cache.view(-1, 2, self.kv.block_size, self.hkv, D)
        ok = slots >= 0
        blk_i, off = slots[ok] // self.kv.block_size, slots[ok] % self.kv.block_size
        flat[blk_i, 0, off] = k[ok]
        flat[blk_i, 1, off] = v[ok]
        a = attend(li, q, k, v)
        x = self._reduce(F.linear(a.reshape(T, self.hq * D), o_w), x)
        gu = F.linear(F.rms_norm(x, (x.shape[-1],), blk.norm2.weight, mc.norm_eps), gu_w)
        return self._reduce(F.linear(F.silu(gu[:, 0::2]) * gu[:, 1::2], dn_w), x)

    def _attend_torch_prefill(self, li, q, k, v, table, start, total):
        """Causal SDPA of a prompt chunk against the pages gathered by indexing (comparison arm)."""
        D, n = self.mc.head_dim, q.shape[0]
        if start > 0:
            nb = (total + self.kv.block_size - 1) // self.kv.block_size
            c = self.kv.caches[li].view(-1, 2, self.kv.block_size, self.hkv, D)[table[0, :nb].long()]
            k = c[:, 0].reshape(-1, self.hkv, D)[:total]
            v = c[:, 1].reshape(-1, self.hkv, D)[:total]
        qh, kh, vh = q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None]
        if start == 0:
            o = F.scaled_dot_product_attention(qh, kh, vh, is_causal=True, enable_gqa=self.hq != self.hkv)
        else:
            mask = torch.arange(total, device=q.device)[None, :] <= (start + torch.arange(n, device=q.device))[:, None]
            o = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask, enable_gqa=self.hq != self.hkv)
        return o[0].transpose(0, 1).contiguous()

    def _attend_torch_decode(self, li, q, table, lens, max_len):
        """One query row per sequence against its pages: gather [B, L, Hkv, D] by indexing the block table, SDPA
        with a length mask (comparison arm)."""
        D, B = self.mc.head_dim, q.shape[0]
        nb = (max_len + self.kv.block_size - 1) // self.kv.block_size
        c = self.kv.caches[li].view(-1, 2, self.kv.block_size, self.hkv, D)[table[:, :nb].long()]   # [B, nb, 2, bs, Hkv, D]
        kk = c[:, :, 0].reshape(B, nb * self.kv.block_size, self.hkv, D).transpose(1, 2)
        vv = c[:, :, 1].reshape(B, nb * self.kv.block_size, self.hkv, D).transpose(1, 2)
        mask = (torch.arange(nb * self.kv.block_size, device=q.device)[None, :] < lens[:, None].long())[:, None, None, :]
        o = F.scaled_dot_product_attention(q[:, :, None, :], kk, vv, attn_mask=mask, enable_gqa=self.hq != self.hkv)
        return o[:, :, 0, :]

    def _embed(self, ids: torch.Tensor) -> torch.Tensor:
        tp = self.tp
        if self.native and tp is not None and tp.world > 1 and tp.fused and hasattr(self.m.embed, "local_v"):
            # vocabulary-parallel lookup summed over the ranks by the in-kernel-synchronised all-reduce (a staging
            # buffer of its own: used once per step, far from its previous use)
            emb = self.m.embed
            T, d = ids.numel(), self.mc.d_model
            cap = max(self.cfg.max_batch, self.cfg.prefill_chunk, self.cfg.max_prefill_tokens)
            buf = tp.symm_buffer("serve.embed", (cap * d * 2 + 255) // 256 * 256)
            stage = buf.view(torch.bfloat16, T * d).view(T, d)
            flat = ids.reshape(-1)
            mask = (flat >= emb.lo) & (flat < emb.lo + emb.local_v)
            local = (flat - emb.lo).clamp(0, emb.local_v - 1)
            stage.copy_(F.embedding(local, emb.weight) * mask[:, None].to(emb.weight.dtype))
            out = torch.empty(T, d, dtype=torch.bfloat16, device=ids.device)
            tp.symm.all_reduce_one_shot_sync(buf, out, T * d)
            return out.view(*ids.shape, d)
        return self.m.embed(ids)

    def _logits_argmax(self, x_last: torch.Tensor) -> torch.Tensor:
        mc = self.mc
        if self.native:
            h, _, _ = native.norm_fwd(x_last.contiguous(), self.m.norm_f.weight, None, mc.norm_eps, True, want_stats=False)
            logits = gemm(h, self.m.lm_head)
            if self.tp is not None and self.tp.world > 1 and self.tp.fused:
                cand = self.tp.symm_buffer("serve.argmax", max(self.cfg.max_batch, 1) * 8)
                return self.tp.symm.tp_argmax(logits, self.tp.rank * logits.shape[1], mc.vocab_size, cand)
            if self.tp is not None and self.tp.world > 1:
                full = self.tp.pg.all_gather(logits, dim=-1)
                return full[:, :mc.vocab_size].float().argmax(-1)
            return native.argmax_rows(logits, mc.vocab_size)
        h, _ = reference.rms_norm_ref(x_last, self.m.norm_f.weight, mc.norm_eps)
        logits = F.linear(h.to(x_last.dtype), self.m.lm_head)
        if self.tp is not None and self.tp.world > 1:
            logits = self.tp.pg.all_gather(logits, dim=-1)
        return logits[:, :mc.vocab_size].float().argmax(-1)

    # ---- prefill of one request chunk
    @torch.no_grad()
    def _prefill(self, r: Request) -> Optional[int]:
        start = r.prefilled
        chunk = r.prompt_tokens[start:start + self.cfg.prefill_chunk]
        n = len(chunk)
        slots, _ = self.kv.append_tokens(r.id, n)
        if slots is None:
            raise MemoryError(f"KV cache exhausted while prefilling request {r.id}")
        dev = self.device
        ids = torch.tensor(chunk, dtype=torch.int64, device=dev)
        pos = torch.arange(start, start + n, dtype=torch.int64, device=dev)
        slots = slots.to(dev)
        table, _ = self.kv.build_tables([r.id], self.max_blocks, dev)
        total = start + n

        paged_prefill = self.native and start > 0 and self.kv.block_size == 16

        def attend(li, q, k, v):
            if paged_prefill:
                # a later chunk: K / V of the cached prefix and of this chunk are read page by page through the
                # block table inside the attention kernel (the chunk's own rows were written by the block just before)
                return native.flash_fwd_paged(q, self.kv.caches[li], table, 1, n, total, causal=True)
            if start == 0:
                kk, vv = k, v
            elif self.native:
                kk, vv = native.kv_gather(self.kv.caches[li], table[0], total)
            else:
                nb = (total + self.kv.block_size - 1) // self.kv.block_size
                c = self.kv.caches[li][table[0, :nb].long()]
                kk = c[:, 0].reshape(-1, self.hkv, self.mc.head_dim)[:total]
                vv = c[:, 1].reshape(-1, self.hkv, self.mc.head_dim)[:total]
            if self.native and start == 0:
                out, _ = native.flash_fwd(q, kk, vv, 1, n, causal=True, want_lse=False)
                return out
            if self.native:                  # a later chunk: its rows are the last n positions of the gathered pages
                return native.flash_fwd_prefix(q, kk, vv, 1, n, total, causal=True)
            if self.cfg.torch_ops:
                return self._attend_torch_prefill(li, q, k, v, table, start, total)
            o, _ = reference.attention_ref(q[None], kk[None], vv[None], causal=True, start_pos=start)
            return o[0].to(q.dtype)
        x = self._embed(ids[None])[0]
        for li, blk in enumerate(self.m.blocks):
            x = self._block(li, blk, x, pos, slots, attend)
        r.prefilled = total
        if r.prefilled >= len(r.prompt_tokens):
            return int(self._logits_argmax(x[-1:])[0])
        return None

    # ---- first chunks of several requests in one pass (equal lengths: one batched causal attention)
    @torch.no_grad()
    def _prefill_many(self, reqs: List[Request], n: int) -> Dict[int, int]:
        dev = self.device
        B = len(reqs)
        slot_list = []
        for r in reqs:
            s, _ = self.kv.append_tokens(r.id, n)
            if s is None:
                raise MemoryError(f"KV cache exhausted while prefilling request {r.id}")
            slot_list.append(s)
        ids = torch.tensor([r.prompt_tokens[:n] for r in reqs], dtype=torch.int64, device=dev)
        pos = torch.arange(n, dtype=torch.int64, device=dev).repeat(B)
        slots = torch.cat(slot_list).to(dev)

        def attend(li, q, k, v):
            out, _ = native.flash_fwd(q, k, v, B, n, causal=True, want_lse=False)
            return out
        x = self._embed(ids).reshape(B * n, -1)
        for li, blk in enumerate(self.m.blocks):
            x = self._block(li, blk, x, pos, slots, attend)
        done = []
        for i, r in enumerate(reqs):
            r.prefilled = n
            if r.prefilled >= len(r.prompt_tokens):
                done.append(i)
        if not done:
            return {}
        rows = torch.tensor([i * n + n - 1 for i in done], dtype=torch.int64, device=dev)
        toks = self._logits_argmax(x[rows]).tolist()
        return {reqs[i].id: int(t) for i, t in zip(done, toks)}

    # ---- one decode step for a set of requests
    def _decode_core(self, last, pos, slots, table, lens, max_len: int) -> torch.Tensor:
        """Device-only part of a decode step (no host reads): embed, all blocks, head, arg-max."""
        def attend(li, q, k, v):
            if self.native:
                return native.paged_decode(q, self.kv.caches[li], table, lens, max_len,
                                           split_tokens=self.cfg.decode_split_tokens)
            if self.cfg.torch_ops:
                return self._attend_torch_decode(li, q, table, lens, max_len)
            return reference.paged_attention_ref(q, self.kv.caches[li], table.cpu(), lens.cpu().tolist()).to(q.dtype)
        x = self._embed(last[None])[0]
        for li, blk in enumerate(self.m.blocks):
            x = self._block(li, blk, x, pos, slots, attend)
        return self._logits_argmax(x)

    @staticmethod
    def _bucket(n: int, lo: int = 1) -> int:
        b = lo
        while b < n:
            b *= 2
        return b

    @torch.no_grad()
    def _decode(self, reqs: List[Request]) -> List[int]:
        dev = self.device
        B = len(reqs)
        last_l = [r.generated[-1] if r.generated else r.prompt_tokens[-1] for r in reqs]
        lens_before = [self.kv.get_sequence_length(r.id) for r in reqs]
        slot_list = []
        for r in reqs:
            s, _ = self.kv.append_tokens(r.id, 1)
            if s is None:
                raise MemoryError(f"KV cache exhausted while decoding request {r.id}")
            slot_list.append(s)
        table, lens = self.kv.build_tables([r.id for r in reqs], self.max_blocks, dev)
        max_len = max(lens_before) + 1
        if self._graphs is None:
            last = torch.tensor(last_l, dtype=torch.int64, device=dev)
            slots = torch.cat(slot_list).to(dev)
            pos = torch.tensor(lens_before, dtype=torch.int64, device=dev)
            return self._decode_core(last, pos, slots, table, lens, max_len).tolist()
        # Graph path: pad the batch to a power of two and the length bound to a multiple of 512 so that a
        # handful of captured graphs covers every step. Padding rows write nowhere (slot -1) and attend to
        # one token of block 0; their outputs are dropped.
        Bp = self._bucket(B)
        Lp = min(self._bucket(max_len, 512), max(self.cfg.max_seq_len, 512))
        pad = Bp - B
        host = torch.empty(3, Bp, dtype=torch.int64, pin_memory=True)
        host[0, :B] = torch.tensor(last_l, dtype=torch.int64)
        host[1, :B] = torch.tensor(lens_before, dtype=torch.int64)
        host[2, :B] = torch.cat(slot_list).to(torch.int64).cpu()
        if pad:
            host[0, B:] = 0
            host[1, B:] = 0
            host[2, B:] = -1
        devt = host.to(dev, non_blocking=True)
        if pad:
            table = torch.cat([table, table.new_zeros(pad, table.shape[1])], 0)
            lens = torch.cat([lens, lens.new_ones(pad)], 0)
        fn = lambda a, b_, c, t, l: self._decode_core(a, b_, c, t, l, Lp)
        out = self._graphs.run(f"decode_L{Lp}", fn, devt[0], devt[1], devt[2], table.contiguous(), lens.contiguous())
        return out[:B].tolist()

    # ---- scheduler entry point
    def execute_batch(self, batch: Batch) -> BatchOutput:
        out: Dict[int, int] = {}
        singles = list(batch.prefill)
        if self.native and len(singles) > 1:
            # group the requests that start their prompt now by the length of their first chunk
            groups: Dict[int, List[Request]] = {}
            for r in singles:
                if r.prefilled == 0:
                    groups.setdefault(min(len(r.prompt_tokens), self.cfg.prefill_chunk), []).append(r)
            singles = [r for r in singles if r.prefilled != 0]
            for n, rs in groups.items():
                per = max(1, self.cfg.max_prefill_tokens // max(n, 1))
                for i in range(0, len(rs), per):
                    part = rs[i:i + per]
                    if len(part) == 1 or n < 1:
                        singles.extend(part)
                    else:
                        out.update(self._prefill_many(part, n))
        for r in singles:
            tok = self._prefill(r)
            if tok is not None:
                out[r.id] = tok
        if batch.decode:
            toks = self._decode(batch.decode)
            for r, t in zip(batch.decode, toks):
                out[r.id] = int(t)
        self.tokens_generated += len(out)
        return BatchOutput(out)
