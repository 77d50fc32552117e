"""Non-interleaved 1F1B pipeline schedule over NCCL point-to-point.

Each stage runs ``warm-up forwards -> (forward, backward) pairs -> cool-down backwards``.
Activations and their gradients travel with ``batch_isend_irecv``: the send of one
direction and the receive of the other are issued as one batch per step ("send forward,
receive backward" / "send backward, receive forward"), in the same order on both
neighbours, because NCCL executes a rank's p2p calls towards one peer in issue order.
The calls are ordered against the compute stream by NCCL's own events, so the host
never blocks (the reference follows every p2p call with a device-wide
``torch.cuda.synchronize()``, schedules.py:506-657).  The compute stream waits for a
transfer only where it consumes what was received: a step that only sends (the
activations of the warm-up forwards, the gradients of the cool-down backwards) is left
in flight behind the next forward / backward pass, its payload kept alive until the next
p2p step, where the stream joins it before anything else is posted.

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
        for r in dist.batch_isend_irecv([dist.P2POp(dist.isend, meta, peer)]):
            r.wait()
        self._meta[(tag, peer)] = (tuple(t.shape), t.dtype, t.requires_grad)

    def _exchange_meta_recv(self, peer: int, tag: str):
        if (tag, peer) not in self._meta:
            meta = torch.empty(META_LEN, dtype=torch.int64, device=self.device)
            for r in dist.batch_isend_irecv([dist.P2POp(dist.irecv, meta, peer)]):
                r.wait()
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
        #: send-only steps still in flight: (requests, payload tensors kept alive until joined)
        self._sends_in_flight: List[Tuple[list, list]] = []
        #: set False to wait for every send where it is posted (A/B timing of the overlap)
        self.overlap_sends = True

    def _join_sends(self):
        for reqs, _keep in self._sends_in_flight:
            for r in reqs:
                r.wait()
        self._sends_in_flight = []

    # ---------------------------------------------------------------------- single steps
    def _forward(self, batch: Optional[Dict], k: int, recv):
        if not self.first:
            x = P2PHandler.finish(*recv)
            x.requires_grad_(True)
            self.model.set_input_tensor(x)
        else:
            x = None
        self.engine._micro = k
        if self.engine.pre_unit is not None:      # the first stage; also the decoder stage of an encoder-decoder model
            self.engine._wait_params(self.engine.pre_unit)
        if self.last:
            out = self.model(**batch)
        else:
            kwargs = {k2: v for k2, v in batch.items() if k2 != "labels"}
            res = self.model(**kwargs)
            if isinstance(res, tuple):
                hidden, residual = res
                out = hidden if residual is None else hidden + residual
            else:
                out = res      # already one tensor (normalised output of an encoder's last block)
        return x, out

    def _backward(self, x, out, k: int, grad):
        self.engine._micro = k
        self.engine._wait_bucket(self.engine.pre_unit)
        self.engine._wait_bucket(self.engine.post_unit)
        if self.last:
            self.engine.scaler.scale(out).backward()
        else:
            torch.autograd.backward(out, grad)
        if self.engine.pre_unit is not None:
            self.engine._unit_backward_done(self.engine.pre_unit)
        return None if x is None else x.grad

    # -------------------------------------------------------------------------- schedule
    def _exchange(self, send_fwd=None, send_bwd=None, recv_fwd=False, recv_bwd=False):
        """One batched p2p step.  Sends and receives that belong together are issued in a
        single ``batch_isend_irecv`` per neighbour pair, in the same order on both sides
        (NCCL runs a rank's p2p calls towards one peer in issue order, so un-paired calls
        on the two sides deadlock).  Returns (received forward input, received gradient)."""
        ps = self.ps
        self._join_sends()
        ops, keep, slots = [], [], {}
        if send_fwd is not None and not self.last:
            for peer, info in ps.send_next:
                part = (send_fwd[info.slice_of(send_fwd.shape[0])] if info.is_sharded else send_fwd).contiguous()
                self.p2p._exchange_meta_send(peer, part, "fwd")
                ops.append(dist.P2POp(dist.isend, part, peer))
                keep.append(part)
        if recv_bwd and not self.last:
            slots["bwd"] = []
            for peer, info in ps.recv_next:
                shape, dtype, _ = self.p2p._meta[("fwd", peer)]       # gradient has the shape of what was sent
                buf = torch.empty(shape, dtype=dtype, device=self.device)
                slots["bwd"].append((info, buf))
                ops.append(dist.P2POp(dist.irecv, buf, peer))
        if send_bwd is not None and not self.first:
            for peer, info in ps.send_prev:
                part = (send_bwd[info.slice_of(send_bwd.shape[0])] if info.is_sharded else send_bwd).contiguous()
                ops.append(dist.P2POp(dist.isend, part, peer))
                keep.append(part)
        if recv_fwd and not self.first:
            slots["fwd"] = []
            for peer, info in ps.recv_prev:
                shape, dtype, _ = self.p2p._exchange_meta_recv(peer, "fwd")
                buf = torch.empty(shape, dtype=dtype, device=self.device)
                slots["fwd"].append((info, buf))
                ops.append(dist.P2POp(dist.irecv, buf, peer))
        if ops:
            reqs = dist.batch_isend_irecv(ops)
            if not slots and self.overlap_sends:
                self._sends_in_flight.append((reqs, keep))     # nothing to consume: let it run behind the next pass
            else:
                for r in reqs:
                    r.wait()

        def assemble(parts):
            """Concatenates batch slices in slice order.  Several peers may return the same slice
            (the tensor-parallel ranks of the next stage all hold the gradient of what this rank
            sent them): one copy per slice is kept."""
            if not parts:
                return None
            by_slice = {}
            for info, buf in parts:
                by_slice.setdefault(info.shard_idx if info.is_sharded else 0, buf)
            if len(by_slice) == 1:
                return next(iter(by_slice.values()))
            return torch.cat([by_slice[k] for k in sorted(by_slice)], dim=0)

        return assemble(slots.get("fwd", [])), assemble(slots.get("bwd", []))

    def train_step(self, batches: List[Dict]) -> torch.Tensor:
        G, W = self.G, self.num_warmup
        remaining = G - W
        inflight: List[Tuple] = []       # (input, output, micro index)
        losses = []
        f = 0

        def fwd(x_in):
            nonlocal f
            x, out = self._forward(batches[f], f, None if x_in is None else ([], x_in))
            inflight.append((x, out, f))
            f += 1
            return out

        def bwd(grad):
            x0, out0, k0 = inflight.pop(0)
            if self.last:
                losses.append(out0.detach())
            return self._backward(x0, out0, k0, grad)

        # warm-up: receive, forward, send
        for i in range(W):
            x_in, _ = self._exchange(recv_fwd=True)
            out = fwd(x_in)
            self._exchange(send_fwd=out.detach())
        x_in = None
        if remaining > 0:
            x_in, _ = self._exchange(recv_fwd=True)
        # steady state: forward, (send forward | receive gradient), backward, (send gradient | receive next)
        for i in range(remaining):
            out = fwd(x_in)
            _, grad = self._exchange(send_fwd=None if self.last else out.detach(), recv_bwd=True)
            gx = bwd(grad)
            if i + 1 < remaining:
                x_in, _ = self._exchange(send_bwd=gx, recv_fwd=True)
            else:
                self._exchange(send_bwd=gx)
        # cool-down
        while inflight:
            _, grad = self._exchange(recv_bwd=True)
            gx = bwd(grad)
            self._exchange(send_bwd=gx)
        self._join_sends()
        self.engine.flush_tied()
        if self.last:
            return torch.stack(losses).mean()
        return torch.zeros((), device=self.device)
