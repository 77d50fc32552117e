"""Non-interleaved 1F1B pipeline schedule over NCCL point-to-point.

Each stage runs ``warm-up forwards -> (forward, backward) pairs -> cool-down backwards``.
Activations and their gradients travel with ``batch_isend_irecv``; the calls are ordered
against the compute stream by NCCL's own events, so nothing waits on the host: receives
for the next step are posted before the current step's compute is launched and the
compute stream only blocks when it really needs the data (the reference follows every
p2p call with a device-wide ``torch.cuda.synchronize()``, schedules.py:506-657).

Stage boundary tensor: a stage hands on ``hidden + residual`` as one ``[b, s, h]`` tensor
(one add), and the next stage starts with ``residual = None``; this is the same math as
passing the pair and halves the p2p volume.  Heterogeneous neighbours (different micro
batch / dp) slice or concatenate along the batch dimension as the rank plan's
:class:`~mist_b200.parallel.state.ShardInfo` routes say.  Tensor metadata is exchanged once
per route (ndim, dims, dtype) before the first payload.

Parity: reference mist/pipeline_parallel/schedules.py:171-286 (forward / backward step),
:364-469 (send / recv helpers), :675-921 (P2PHandler, metadata encoding :848-884),
:924-1138 (schedule).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .state import ShardInfo

_DTYPE_CODES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2, torch.int64: 3}
_CODE_DTYPES = {v: k for k, v in _DTYPE_CODES.items()}
META_LEN = 9      # ndim, up to 6 dims, dtype code, requires_grad


def encode_meta(t: torch.Tensor) -> List[int]:
    dims = list(t.shape)
    assert len(dims) <= 6, "p2p tensors have at most 6 dimensions"
    return [len(dims)] + dims + [0] * (6 - len(dims)) + [_DTYPE_CODES[t.dtype], int(t.requires_grad)]


def decode_meta(vec: List[int]) -> Tuple[Tuple[int, ...], torch.dtype, bool]:
    n = int(vec[0])
    return tuple(int(x) for x in vec[1:1 + n]), _CODE_DTYPES[int(vec[7])], bool(vec[8])


class P2PHandler:
    """Sends / receives one activation-shaped tensor along the forward or backward routes."""

    def __init__(self, pstate, device):
        self.ps = pstate
        self.device = device
        self._meta: Dict[Tuple[str, int], Tuple] = {}

    def _exchange_meta_send(self, peer: int, t: torch.Tensor, tag: str):
        if (tag, peer) in self._meta:
            return
        meta = torch.tensor(encode_meta(t), dtype=torch.int64, device=self.device)
        dist.send(meta, peer)
        self._meta[(tag, peer)] = (tuple(t.shape), t.dtype, t.requires_grad)

    def _exchange_meta_recv(self, peer: int, tag: str):
        if (tag, peer) not in self._meta:
            meta = torch.empty(META_LEN, dtype=torch.int64, device=self.device)
            dist.recv(meta, peer)
            self._meta[(tag, peer)] = decode_meta(meta.tolist())
        return self._meta[(tag, peer)]

    def send(self, t: torch.Tensor, routes: List[Tuple[int, ShardInfo]], tag: str):
        """Posts the sends of ``t`` (sliced per route); returns the request handles."""
        ops, keep = [], []
        for peer, info in routes:
            part = t[info.slice_of(t.shape[0])] if info.is_sharded else t
            part = part.contiguous()
            self._exchange_meta_send(peer, part, tag)
            ops.append(dist.P2POp(dist.isend, part, peer))
            keep.append(part)
        reqs = dist.batch_isend_irecv(ops) if ops else []
        return reqs, keep

    def recv(self, routes: List[Tuple[int, ShardInfo]], tag: str):
        """Posts the receives; returns (handles, tensor).  Several senders fill batch slices."""
        parts, ops = [], []
        for peer, info in routes:
            shape, dtype, _ = self._exchange_meta_recv(peer, tag)
            buf = torch.empty(shape, dtype=dtype, device=self.device)
            parts.append((info, buf))
            ops.append(dist.P2POp(dist.irecv, buf, peer))
        reqs = dist.batch_isend_irecv(ops) if ops else []
        if len(parts) == 1:
            return reqs, parts[0][1]
        parts.sort(key=lambda x: x[0].shard_idx)
        return reqs, parts      # concatenated after the wait

    @staticmethod
    def finish(reqs, payload):
        for r in reqs:
            r.wait()
        if isinstance(payload, list):
            return torch.cat([b for _, b in payload], dim=0)
        return payload


class PipelineSchedule:
    def __init__(self, session):
        self.session = session
        self.ps = session.ps
        self.engine = session.engine
        self.model = session.model
        self.device = session.device
        self.G = session.G
        self.p2p = P2PHandler(self.ps, self.device)
        self.first, self.last = self.ps.is_first_stage, self.ps.is_last_stage
        S = self.ps.num_stages
        self.num_warmup = min(S - 1 - self.ps.stage, self.G)

    # ---------------------------------------------------------------------- single steps
    def _forward(self, batch: Optional[Dict], k: int, recv):
        if not self.first:
            x = P2PHandler.finish(*recv)
            x.requires_grad_(True)
            self.model.set_input_tensor(x)
        else:
            x = None
        self.engine._micro = k
        if self.first and self.engine.pre_unit is not None:
            self.engine._wait_params(self.engine.pre_unit)
        if self.last:
            kwargs = dict(batch)
            if not self.first:
                kwargs["input_ids"] = batch["input_ids"]   # only the shape is used past stage 0
            out = self.model(**kwargs)
        else:
            kwargs = {k2: v for k2, v in batch.items() if k2 != "labels"}
            hidden, residual = self.model(**kwargs)
            out = hidden if residual is None else hidden + residual
        return x, out

    def _backward(self, x, out, k: int, grad):
        self.engine._micro = k
        self.engine._wait_bucket(self.engine.pre_unit)
        self.engine._wait_bucket(self.engine.post_unit)
        if self.last:
            out.backward()
        else:
            torch.autograd.backward(out, grad)
        if self.engine.pre_unit is not None:
            self.engine._unit_backward_done(self.engine.pre_unit)
        return None if x is None else x.grad

    # -------------------------------------------------------------------------- schedule
    def train_step(self, batches: List[Dict]) -> torch.Tensor:
        G, W = self.G, self.num_warmup
        ps = self.ps
        pending_sends = []
        inflight: List[Tuple] = []       # (input, output, micro index)
        losses = []
        f = b = 0

        def post_recv_fwd():
            return self.p2p.recv(ps.recv_prev, "fwd") if not self.first else None

        def post_recv_bwd():
            return self.p2p.recv(ps.recv_next, "bwd") if not self.last else None

        def send_fwd(t):
            if not self.last:
                pending_sends.append(self.p2p.send(t.detach(), ps.send_next, "fwd"))

        def send_bwd(g):
            if not self.first and g is not None:
                pending_sends.append(self.p2p.send(g, ps.send_prev, "bwd"))

        recv_f = post_recv_fwd() if G > 0 else None
        # warm-up forwards
        for _ in range(W):
            x, out = self._forward(batches[f], f, recv_f)
            recv_f = post_recv_fwd() if f + 1 < G else None
            send_fwd(out)
            inflight.append((x, out, f))
            f += 1
        # steady state: one forward, one backward
        recv_b = post_recv_bwd() if (f < G or inflight) else None
        while f < G:
            x, out = self._forward(batches[f], f, recv_f)
            recv_f = post_recv_fwd() if f + 1 < G else None
            send_fwd(out)
            inflight.append((x, out, f))
            f += 1
            x0, out0, k0 = inflight.pop(0)
            grad = P2PHandler.finish(*recv_b) if recv_b is not None else None
            if self.last:
                losses.append(out0.detach())
            gx = self._backward(x0, out0, k0, grad)
            b += 1
            recv_b = post_recv_bwd() if (b < G) else None
            send_bwd(gx)
        # cool-down backwards
        while inflight:
            x0, out0, k0 = inflight.pop(0)
            grad = P2PHandler.finish(*recv_b) if recv_b is not None else None
            if self.last:
                losses.append(out0.detach())
            gx = self._backward(x0, out0, k0, grad)
            b += 1
            recv_b = post_recv_bwd() if (b < G) else None
            send_bwd(gx)
        for reqs, keep in pending_sends:
            for r in reqs:
                r.wait()
        if self.last:
            return torch.stack(losses).mean()
        return torch.zeros((), device=self.device)
