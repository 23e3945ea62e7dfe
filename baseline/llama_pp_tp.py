"""Plain torch.distributed pipeline x tensor-parallel Llama training step: the model cut into ``pp`` stages of
Megatron-style tensor-parallel blocks (``llama_tp.Block``: cuBLAS linears, SDPA, NCCL all-reduce after each
row-parallel linear), a 1F1B schedule over micro-batches of one sequence with full recomputation of the stage
forward in the backward pass, stage activations over NCCL send / recv, fused torch AdamW per stage. The comparison
arm for the pipeline configuration; none of this package's kernels run here.

Ranks are laid out with the tensor-parallel index fastest: rank = stage * tp + tp_rank."""
import torch
import torch.distributed as dist
import torch.nn as nn

import llama_tp as L


class Stage(nn.Module):
    def __init__(self, c, tp, tp_rank, lo, hi, first, last, dev):
        super().__init__()
        kw = dict(device=dev, dtype=torch.bfloat16)
        V = (c["vocab_size"] + 127) // 128 * 128
        self.Vl, self.tp_rank, self.first, self.last = V // tp, tp_rank, first, last
        self.embed = nn.Embedding(self.Vl, c["d_model"], **kw) if first else None
        self.blocks = nn.ModuleList([L.Block(c, tp, dev) for _ in range(lo, hi)])
        self.nf = nn.RMSNorm(c["d_model"], eps=c.get("norm_eps", 1e-5), **kw) if last else None
        self.head = nn.Linear(c["d_model"], self.Vl, bias=False, **kw) if last else None

    def forward(self, x, tgt=None):
        lo = self.tp_rank * self.Vl
        if self.first:
            mask = (x >= lo) & (x < lo + self.Vl)
            x = L._AllReduce.apply(self.embed((x - lo).clamp(0, self.Vl - 1)) * mask[..., None])
        for b in self.blocks:
            x = b(x)
        if not self.last:
            return x
        logits = self.head(L._CopyIn.apply(self.nf(x))).float()
        m = logits.detach().amax(-1)
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=L.GROUP)
        se = L._AllReduce.apply((logits - m[..., None]).exp().sum(-1))
        tmask = (tgt >= lo) & (tgt < lo + self.Vl)
        tl = L._AllReduce.apply(logits.gather(-1, (tgt - lo).clamp(0, self.Vl - 1)[..., None])[..., 0] * tmask)
        return (m + se.log() - tl).mean()


def build(cfg, dev, ids, tgt, pp, tp, micro_batches):
    """Returns (step, n_params_of_this_rank). ``ids`` / ``tgt`` are [micro_batches, seq]."""
    W, rank = dist.get_world_size(), dist.get_rank()
    assert pp * tp == W
    stage_i, tp_rank = rank // tp, rank % tp
    for s in range(pp):                                   # every rank creates every group, in the same order
        g = dist.new_group(list(range(s * tp, (s + 1) * tp)))
        if s == stage_i:
            L.GROUP = g
    n = cfg["n_layers"]
    per, extra = divmod(n, pp)
    lo = stage_i * per + min(stage_i, extra)
    hi = lo + per + (1 if stage_i < extra else 0)
    first, last = stage_i == 0, stage_i == pp - 1
    mod = Stage(cfg, tp, tp_rank, lo, hi, first, last, dev)
    L.init_weights(mod, cfg)
    opt = torch.optim.AdamW(mod.parameters(), lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, fused=True)
    S, d = ids.shape[1], cfg["d_model"]
    prev_r, next_r = rank - tp, rank + tp
    M = micro_batches

    def exchange(send_t=None, send_to=None, recv_from=None, recv_shape=None):
        """One grouped NCCL exchange: an optional send and an optional receive that progress together (a send
        queued in front of the matching receive of the opposite direction would otherwise block both ranks)."""
        ops, out = [], None
        if send_t is not None:
            ops.append(dist.P2POp(dist.isend, send_t.contiguous(), send_to))
        if recv_from is not None:
            out = torch.empty(recv_shape, device=dev, dtype=torch.bfloat16)
            ops.append(dist.P2POp(dist.irecv, out, recv_from))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        return out

    act = (1, S, d)

    def forward(x):
        """Stage forward without a graph; the input is kept and the forward is recomputed in the backward."""
        if last:
            return None
        with torch.no_grad():
            return mod(x)

    def backward(x, k, gy, losses):
        if not first:
            x = x.requires_grad_(True)
        if last:
            loss = mod(x, tgt[k:k + 1]) / M
            loss.backward()
            losses.append(loss.detach())
        else:
            mod(x).backward(gy)
        return None if first else x.grad

    def step():
        opt.zero_grad(set_to_none=True)
        kept, losses = [], []
        warm = min(pp - 1 - stage_i, M)
        rem = M - warm
        nf = nb = 0                                        # micro-batches whose forward / backward has started

        def recv_forward():
            nonlocal nf
            x = ids[nf:nf + 1] if first else exchange(recv_from=prev_r, recv_shape=act)
            nf += 1
            kept.append(x)
            return x

        for _ in range(warm):
            y = forward(recv_forward())
            exchange(send_t=y, send_to=next_r)
        x = recv_forward() if rem > 0 else None
        for k in range(rem):                               # steady state: one forward, one backward
            y = forward(x)
            gy = None if last else exchange(send_t=y, send_to=next_r, recv_from=next_r, recv_shape=act)
            gx = backward(kept.pop(0), nb, gy, losses)
            nb += 1
            if k == rem - 1:
                if not first:
                    exchange(send_t=gx, send_to=prev_r)
            elif first:
                x = recv_forward()
            else:
                x = exchange(send_t=gx, send_to=prev_r, recv_from=prev_r, recv_shape=act)
                nf += 1
                kept.append(x)
        for _ in range(warm):                              # cool-down
            gy = exchange(recv_from=next_r, recv_shape=act)
            gx = backward(kept.pop(0), nb, gy, losses)
            nb += 1
            if not first:
                exchange(send_t=gx, send_to=prev_r)
        opt.step()
        return torch.stack(losses).sum() if losses else torch.zeros((), device=dev)

    return step, sum(p.numel() for p in mod.parameters())
