"""Data-parallel gradient exchange for end-to-end training: bucket plan and staged all-reduce.

Mirrors the reference's distributed step (gpu/distributed_step.cpp):

* ``build_gradient_bucket_plan`` - gradients in weight order packed into flat fp32 buckets of a target size
  (32 MiB by default, gpu/distributed_step.h:14), with the same closing rule and the same FNV-1a digest
  (gpu/distributed_step.cpp:61-118) so that ranks can check that they agree on the layout;
* ``staged_gradient_allreduce`` - the stages of ``prepare_distributed_staged_gradients`` (:120-249): non-finite
  entries zeroed, gradients turned into numerators, bad flag and loss denominator agreed on across ranks, one sum
  per bucket, division by the global denominator, then ``sanitize_and_clip_gradients``
  (gpu/optimizer_step_guard.cpp:76-104).

What differs from the reference is how the three kinds of collectives are issued.  The reference runs an ``all_max``
of the bad flag, then an ``all_sum`` of the denominator, each followed by a host read, before the bucket sums.  On
NVLink those two scalar collectives cost two launch latencies and two host round trips and move eight bytes, so
here both scalars ride in two extra slots at the tail of the last bucket (the flag as a 0/1 count, which a sum
reduces just as well as a max), every bucket is all-reduced asynchronously on the communication stream in plan
order, and the host reads the two scalars once, after the last bucket.  The decisions taken from them (skip the
step when any rank is bad, report a zero denominator) are the reference's.  The collective itself is plain
``torch.distributed.all_reduce`` (NCCL on GPUs, in-switch reduction where NCCL enables it; gloo in the CPU tests).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

DEFAULT_BUCKET_BYTES = 32 * 1024 * 1024  # kDefaultGradientBucketBytes, gpu/distributed_step.h:14
_INT_MAX = 2 ** 31 - 1
_FNV_OFFSET = 1469598103934665603
_FNV_PRIME = 1099511628211
_MASK64 = (1 << 64) - 1


@dataclass
class BucketEntry:
    weight_index: int
    offset: int          # in elements, inside the bucket
    elements: int
    shape: tuple


@dataclass
class Bucket:
    elements: int = 0
    bytes: int = 0
    entries: List[BucketEntry] = field(default_factory=list)


@dataclass
class GradientBucketPlan:
    target_bytes: int
    total_bytes: int
    digest: int
    buckets: List[Bucket]


def _hash_word(h: int, value: int) -> int:
    """FNV-1a over the 8 little-endian bytes of ``value`` (hash_word, gpu/distributed_step.cpp:38-44)."""
    for i in range(8):
        h ^= (value >> (8 * i)) & 0xFF
        h = (h * _FNV_PRIME) & _MASK64
    return h


def build_gradient_bucket_plan(shapes: Sequence[Sequence[int]], target_bytes: int = DEFAULT_BUCKET_BYTES) -> GradientBucketPlan:
    """Buckets in weight order.  A bucket is closed before an entry that would take it past ``target_bytes`` (a single
    larger entry gets a bucket of its own) or past the int32 element range - gpu/distributed_step.cpp:61-100."""
    if target_bytes <= 0:
        raise ValueError("gradient bucket target must be positive")
    buckets: List[Bucket] = []
    cur = Bucket()
    total = 0
    for i, shape in enumerate(shapes):
        shape = tuple(int(s) for s in shape)
        elements = int(math.prod(shape)) if shape else 1
        if elements > _INT_MAX:
            raise ValueError("gradient bucket entry exceeds the 32-bit slice index range")
        nbytes = elements * 4
        exceeds_target = cur.bytes > target_bytes or nbytes > target_bytes - min(cur.bytes, target_bytes)
        exceeds_range = cur.elements > _INT_MAX - elements
        if cur.entries and (exceeds_target or exceeds_range):
            buckets.append(cur)
            cur = Bucket()
        cur.entries.append(BucketEntry(i, cur.elements, elements, shape))
        cur.elements += elements
        cur.bytes += nbytes
        total += nbytes
    if cur.entries:
        buckets.append(cur)
    h = _FNV_OFFSET
    for word in (target_bytes, total, len(buckets)):
        h = _hash_word(h, word)
    for b in buckets:
        h = _hash_word(h, b.bytes)
        h = _hash_word(h, len(b.entries))
        for e in b.entries:
            for word in (e.weight_index, e.offset, e.elements, len(e.shape), *e.shape):
                h = _hash_word(h, word)
    return GradientBucketPlan(target_bytes, total, h, buckets)


class BucketStorage:
    """Flat fp32 buffers of a plan on one device, with one view per weight.  A trainer that writes its gradients
    straight into ``views`` needs no packing copy.  Two extra slots carry the packed scalars through the sums: the
    loss denominator rides behind the FIRST bucket (every later bucket can then be finalized as soon as its own sum
    has arrived), the bad flag behind the LAST one (it is only complete once every bucket has been looked at)."""

    def __init__(self, plan: GradientBucketPlan, device):
        self.plan = plan
        self.flat: List[torch.Tensor] = []
        self.views: List[Optional[torch.Tensor]] = [None] * sum(len(b.entries) for b in plan.buckets)
        last = len(plan.buckets) - 1
        for bi, b in enumerate(plan.buckets):
            extra = (1 if bi == 0 else 0) + (1 if bi == last else 0)
            buf = torch.zeros(b.elements + extra, dtype=torch.float32, device=device)
            self.flat.append(buf)
            for e in b.entries:
                self.views[e.weight_index] = buf[e.offset:e.offset + e.elements].view(e.shape)

    @property
    def denominator(self) -> torch.Tensor:
        """The loss-denominator slot (one element) behind the first bucket."""
        n = self.plan.buckets[0].elements
        return self.flat[0][n:n + 1]

    @property
    def bad(self) -> torch.Tensor:
        """The bad-flag slot (one element): the last element of the last bucket."""
        return self.flat[-1][-1:]


@dataclass
class StagedGradientResult:
    gradient_nonfinite: float    # non-finite entries found after the reduction (or the global bad count)
    zero_denominator: bool
    globally_bad: bool
    denominator: float
    buckets: int
    bytes_reduced: int


def sanitize_and_clip_(grads: Sequence[torch.Tensor], max_grad_norm: float) -> torch.Tensor:
    """In place: non-finite entries -> 0, then global-norm clipping; the scale is 0 when anything was non-finite
    (gpu/optimizer_step_guard.cpp:76-104).  Returns the non-finite count (a 0-d tensor)."""
    dev = grads[0].device
    nonfinite = torch.zeros((), dtype=torch.float32, device=dev)
    norm_sq = torch.zeros((), dtype=torch.float32, device=dev)
    for g in grads:
        fin = torch.isfinite(g)
        nonfinite += (~fin).sum().float()
        g.masked_fill_(~fin, 0.0)
        norm_sq += g.float().pow(2).sum()
    if max_grad_norm <= 0.0:
        return nonfinite
    norm = norm_sq.sqrt()
    ordinary = torch.clamp(max_grad_norm / (norm + 1e-6), max=1.0)
    valid = (nonfinite == 0) & torch.isfinite(norm)
    scale = torch.where(valid, ordinary, torch.zeros_like(ordinary))
    torch._foreach_mul_(list(grads), scale)
    return nonfinite


def _all_reduce_buckets(flat, group, comm_stream, dev):
    """One SUM all-reduce per bucket, in plan order, asynchronously; on CUDA on the communication stream."""
    cuda = dev.type == "cuda"
    works = []
    if cuda and comm_stream is not None:
        comm_stream.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(comm_stream):
            for buf in flat:
                works.append(dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group, async_op=True))
    else:
        for buf in flat:
            works.append(dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group, async_op=True))
    for w in works:
        w.wait()
    if cuda and comm_stream is not None:
        torch.cuda.current_stream(dev).wait_stream(comm_stream)


def staged_gradient_allreduce(grads: List[torch.Tensor], loss: torch.Tensor, loss_normalizer: float,
                              gradients_are_numerators: bool, max_grad_norm: float, plan: GradientBucketPlan,
                              storage: Optional[BucketStorage] = None, group=None,
                              comm_stream: Optional["torch.cuda.Stream"] = None) -> StagedGradientResult:
    """Replaces ``grads[i]`` by the globally averaged, clipped gradient (views into ``storage``).

    ``grads`` may already be the views of ``storage`` (no packing copy then).  On CUDA every element-wise stage is
    one fused pass per bucket of the library's kernels (mxb_dp_sanitize / _finalize / _scale), the bucket
    all-reduces are enqueued on ``comm_stream`` (default: the current stream) one after the other in plan order,
    each bucket is finalized behind its own sum while the later sums are in flight, and the host reads the device
    once, at the end.
    CPU tensors (the gloo tests of the host logic) take the same stages through torch ops."""
    if not grads or not plan.buckets:
        raise ValueError("distributed gradient bucket plan is empty")
    dev = grads[0].device
    if storage is None:
        storage = BucketStorage(plan, dev)
    denominator_valid = math.isfinite(loss_normalizer) and loss_normalizer >= 0.0
    safe = float(loss_normalizer) if denominator_valid else 0.0
    for i, g in enumerate(grads):  # pack into the flat buckets when the gradients live elsewhere
        view = storage.views[i]
        if g.data_ptr() != view.data_ptr():
            view.copy_(g.to(torch.float32).reshape(view.shape))
    for i in range(len(grads)):
        grads[i] = storage.views[i]
    cuda = dev.type == "cuda"
    scale = 1.0 if gradients_are_numerators else safe
    nbytes = sum(b.numel() * 4 for b in storage.flat)
    storage.denominator.fill_(safe)  # behind the first bucket, so that its sum can leave right after its own pass
    # -- numerator conversion: non-finite -> 0 (and flagged), x scale
    if cuda:
        from . import _lib
        import ctypes as C
        l = _lib.lib()
        st = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        aux = torch.zeros(4 + l.mxb_dp_partial_floats(), dtype=torch.float32, device=dev)  # flag, totals[3], partials
        P = lambda t, off=0: C.c_void_p(t.data_ptr() + 4 * off)
        # every bucket but the last leaves for its sum right behind its own pass (the last one carries the bad flag,
        # which is complete only after all passes)
        cur = torch.cuda.current_stream(dev)
        comm = comm_stream if comm_stream is not None else cur
        works = []
        with torch.cuda.device(dev):
            for i, (b, buf) in enumerate(zip(plan.buckets, storage.flat)):
                _lib.check(l.mxb_dp_sanitize(P(buf), b.elements, scale, P(aux), st), "mxb_dp_sanitize")
                if i < len(storage.flat) - 1:
                    ev = torch.cuda.Event()
                    ev.record(cur)
                    with torch.cuda.stream(comm):
                        comm.wait_event(ev)
                        works.append(dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group, async_op=True))
        raw_bad = aux[0]
    else:
        raw_bad = torch.zeros((), dtype=torch.float32, device=dev)
        for b, buf in zip(plan.buckets, storage.flat):
            body = buf[:b.elements]
            fin = torch.isfinite(body)
            raw_bad = torch.maximum(raw_bad, (~fin).any().float())
            body.masked_fill_(~fin, 0.0)
            if scale != 1.0:
                body.mul_(scale)
    local_bad = torch.maximum((~torch.isfinite(loss.float())).any().float().to(dev), raw_bad) if safe > 0.0 \
        else torch.zeros((), dtype=torch.float32, device=dev)
    if not denominator_valid:
        local_bad = torch.ones((), dtype=torch.float32, device=dev)
    storage.bad.copy_(local_bad.reshape(1))
    if cuda:
        return _finish_pipelined(storage, plan, group, comm, dev, max_grad_norm, l, st, aux, P, works, nbytes)
    _all_reduce_buckets(storage.flat, group, comm_stream, dev)
    bad_count, denominator = float(storage.bad), float(storage.denominator)  # host read of the two packed scalars
    if bad_count > 0.0:
        return StagedGradientResult(bad_count, False, True, denominator, len(storage.flat), nbytes)
    if not math.isfinite(denominator) or denominator < 0.0:
        raise RuntimeError("distributed global loss denominator is invalid")
    if denominator == 0.0:
        return StagedGradientResult(0.0, True, False, 0.0, len(storage.flat), nbytes)
    # -- divide by the global denominator, sanitize, global norm, clip
    for b, buf in zip(plan.buckets, storage.flat):
        buf[:b.elements].div_(denominator)
    nonfinite = float(sanitize_and_clip_([v for v in storage.views], max_grad_norm))
    return StagedGradientResult(nonfinite, False, False, denominator, len(storage.flat), nbytes)


def _finish_pipelined(storage, plan, group, comm, dev, max_grad_norm, l, st, aux, P, works, nbytes):
    """CUDA: the sums of all buckets but the last are already on the communication stream (each went out behind its own
    sanitize pass); the last one follows now that the bad flag is in place.  On the compute stream every bucket is
    divided, sanitized and measured right behind its own sum, with the divisor taken from the device slot behind the
    first bucket, while the later sums are still in flight.  The host reads the device once, at the end: bad flag,
    denominator, non-finite count."""
    from . import _lib
    cur = torch.cuda.current_stream(dev)
    ready = torch.cuda.Event()
    ready.record(cur)  # every bucket sanitized and the bad flag in its slot
    with torch.cuda.stream(comm):
        comm.wait_event(ready)
        works.append(dist.all_reduce(storage.flat[-1], op=dist.ReduceOp.SUM, group=group, async_op=True))
    with torch.cuda.device(dev):
        for i, (b, buf) in enumerate(zip(plan.buckets, storage.flat)):
            works[i].wait()  # the compute stream waits for this bucket's sum only
            _lib.check(l.mxb_dp_finalize_dev(P(buf), b.elements, P(storage.denominator), float(max_grad_norm), P(aux, 4),
                                             P(aux, 1), st), "mxb_dp_finalize_dev")
        if max_grad_norm > 0.0:
            for b, buf in zip(plan.buckets, storage.flat):
                _lib.check(l.mxb_dp_scale(P(buf), b.elements, P(aux, 3), st), "mxb_dp_scale")
    bad_count, denominator, nonfinite = torch.stack([storage.bad[0], storage.denominator[0], aux[2]]).tolist()
    if bad_count > 0.0:
        return StagedGradientResult(bad_count, False, True, denominator, len(storage.flat), nbytes)
    if not math.isfinite(denominator) or denominator < 0.0:
        raise RuntimeError("distributed global loss denominator is invalid")
    if denominator == 0.0:
        return StagedGradientResult(0.0, True, False, 0.0, len(storage.flat), nbytes)
    return StagedGradientResult(nonfinite, False, False, denominator, len(storage.flat), nbytes)


def hybrid_lm_weight_shapes(layers=12, d_model=1024, heads=16, d_k=64, d_v=64, ffn=4096, vocab=32768) -> List[tuple]:
    """Weight shapes, in weight order, of the end-to-end training configuration: ``layers`` blocks alternating
    gated_deltanet (weights of arch/blocks_gated_deltanet.go:60-101, kv_share off) and attention, each followed by
    a SwiGLU FFN, RMSNorm scales, tied-size embedding and head."""
    key, val = heads * d_k, heads * d_v
    shapes: List[tuple] = [(vocab, d_model)]
    for layer in range(layers):
        if layer % 2 == 0:  # gated_deltanet
            shapes += [(d_model,), (d_model, key), (4, key), (d_model, key), (d_model, val), (4, key), (4, val), (d_model, heads),
                       (heads,), (heads,), (d_model, heads), (d_v,), (d_model, val), (val, d_model)]
        else:               # attention
            shapes += [(d_model,), (d_model, key), (d_model, key), (d_model, val), (val, d_model)]
        shapes += [(d_model,), (d_model, ffn), (d_model, ffn), (ffn, d_model)]
    shapes += [(d_model,), (d_model, vocab)]
    return shapes
