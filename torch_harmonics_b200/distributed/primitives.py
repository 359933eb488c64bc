"""Differentiable all-to-all transposes and the split helpers of the distributed transforms.

Same functions as torch_harmonics/distributed/primitives.py:74-347 and :775-822.  A transpose trades a sharded
axis for a shard of another one: the tensor arrives sharded along ``dims[1]`` (every rank holds a slice of it and
all of ``dims[0]``) and leaves sharded along ``dims[0]`` with ``dims[1]`` complete.  Chunks are balanced and may be
uneven (``compute_split_shapes``).

The exchange itself is ONE ``all_to_all_single`` over NCCL.  Pieces travel in the tensor's own axis order, so that
a transpose costs at most one copy on each side and none on the side whose axis leads (the reference copies every
chunk separately, uses the list form and concatenates).  Backends without all-to-all (gloo, used by the CPU tests)
go through point-to-point sends.
"""

from typing import List

import torch
import torch.distributed as dist

from .utils import azimuth_group, azimuth_group_size, config, is_distributed_azimuth, is_distributed_polar, polar_group, polar_group_size


def compute_split_shapes(size: int, num_chunks: int) -> List[int]:
    """Balanced chunk sizes: the first ``size % num_chunks`` chunks get one extra element.
    Raises RuntimeError when ``size < num_chunks`` (every chunk must be non-empty)."""
    torch._check(size >= num_chunks, lambda: f"Cannot split {size} elements into {num_chunks} chunks; every chunk must be non-empty.")
    base, rem = divmod(size, num_chunks)
    return [base + 1] * rem + [base] * (num_chunks - rem)


def split_tensor_along_dim(tensor, dim, num_chunks):
    """Views of ``tensor`` cut into balanced chunks along ``dim``."""
    torch._check(len(tensor.shape) > dim, lambda: f"Error, tensor dimension is {len(tensor.shape)} which cannot be split along {dim}")
    torch._check(tensor.shape[dim] >= num_chunks, lambda: f"Error, cannot split dim {dim} of size {tensor.shape[dim]} into {num_chunks} chunks. Empty slices are currently not supported.")
    return torch.split(tensor, compute_split_shapes(tensor.shape[dim], num_chunks), dim=dim)


def flatten_and_pad_leading_dims(tensor: torch.Tensor, min_leading_size: int, num_trailing_dims: int = 2):
    """Collapse all but the trailing dims into one leading axis and zero-pad it up to ``min_leading_size``
    (the transposes redistribute this axis, so it must be at least as long as the larger group)."""
    lead_shape = tensor.shape[:-num_trailing_dims]
    tensor = tensor.reshape(-1, *tensor.shape[-num_trailing_dims:])
    lead_size = tensor.shape[0]
    if lead_size < min_leading_size:
        tensor = torch.cat([tensor, tensor.new_zeros((min_leading_size - lead_size, *tensor.shape[1:]))], dim=0)
    return tensor.contiguous(), lead_shape, lead_size


def unpad_and_unflatten_leading_dims(tensor: torch.Tensor, lead_shape, lead_size: int, num_trailing_dims: int = 2) -> torch.Tensor:
    """Inverse of :func:`flatten_and_pad_leading_dims`."""
    tensor = tensor.narrow(0, 0, lead_size)
    return tensor.reshape(*lead_shape, *tensor.shape[-num_trailing_dims:]).contiguous()


def _verify(msg, local_value, expected, group):
    """Debug mode: gather one integer per rank and compare with the expected per-rank list."""
    t = torch.tensor([local_value], dtype=torch.int64)
    if dist.get_backend(group) == "nccl":
        t = t.cuda()
    gathered = [torch.empty_like(t) for _ in range(dist.get_world_size(group))]
    dist.all_gather(gathered, t, group=group)
    got = [int(g.item()) for g in gathered]
    for idx, (a, b) in enumerate(zip(got, expected)):
        if a != b:
            raise ValueError(f"{msg} shapes are not correct. Expected {b}, got {a} for index {idx}. Please check that the number of chunks is correct.")


# Optional record of the exchanges (benchmarking): while a list is installed, every NCCL all-to-all appends
# (bytes sent to other ranks, bytes received from other ranks, start event, end event).
_EXCHANGE_LOG = None


def exchange_log_start():
    """Start recording the all-to-all exchanges of this process (byte counts and CUDA events around each one)."""
    global _EXCHANGE_LOG
    _EXCHANGE_LOG = []


def exchange_log_stop():
    """Stop recording; returns [(bytes_sent, bytes_received, milliseconds)] after synchronising the device."""
    global _EXCHANGE_LOG
    log, _EXCHANGE_LOG = _EXCHANGE_LOG or [], None
    if log:
        torch.cuda.synchronize()
    return [(s, r, e0.elapsed_time(e1)) for s, r, e0, e1 in log]


_SIDE_STREAMS = {}


def _exchange_split(send, send_counts, recv_counts, recv, group):
    """The rank's own block as a device copy on a side stream, the other ranks' blocks as one group of NCCL sends and
    receives: the collective's kernel moves remote bytes only, and the local copy runs beside it at memory speed."""
    me, size = dist.get_rank(group), dist.get_world_size(group)
    ranks = dist.get_process_group_ranks(group)
    soff, roff = [0], [0]
    for a, b in zip(send_counts, recv_counts):
        soff.append(soff[-1] + a)
        roff.append(roff[-1] + b)
    cur = torch.cuda.current_stream(send.device)
    side = _SIDE_STREAMS.get(send.device)
    if side is None:
        side = _SIDE_STREAMS[send.device] = torch.cuda.Stream(device=send.device)
    side.wait_stream(cur)
    with torch.cuda.stream(side):
        recv[roff[me]:roff[me + 1]].copy_(send[soff[me]:soff[me + 1]])
    send.record_stream(side)
    recv.record_stream(side)
    ops = []
    for peer in range(size):
        if peer == me:
            continue
        if send_counts[peer]:
            ops.append(dist.P2POp(dist.isend, send[soff[peer]:soff[peer + 1]], ranks[peer], group))
        if recv_counts[peer]:
            ops.append(dist.P2POp(dist.irecv, recv[roff[peer]:roff[peer + 1]], ranks[peer], group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    cur.wait_stream(side)


def _exchange(send: torch.Tensor, send_counts, recv_counts, group):
    """Flat all-to-all with per-peer element counts."""
    recv = send.new_empty(sum(recv_counts))
    if dist.get_backend(group) == "nccl" and config.exchange == "split" and dist.get_world_size(group) <= config.split_max_group:
        if _EXCHANGE_LOG is not None:
            me = dist.get_rank(group)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        _exchange_split(send, send_counts, recv_counts, recv, group)
        if _EXCHANGE_LOG is not None:
            e1.record()
            es = send.element_size()
            _EXCHANGE_LOG.append(((sum(send_counts) - send_counts[me]) * es, (sum(recv_counts) - recv_counts[me]) * es, e0, e1))
        return recv
    if dist.get_backend(group) == "nccl":
        if _EXCHANGE_LOG is not None:
            me = dist.get_rank(group)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        dist.all_to_all_single(recv, send, output_split_sizes=list(recv_counts), input_split_sizes=list(send_counts), group=group)
        if _EXCHANGE_LOG is not None:
            e1.record()
            es = send.element_size()
            _EXCHANGE_LOG.append(((sum(send_counts) - send_counts[me]) * es, (sum(recv_counts) - recv_counts[me]) * es, e0, e1))
        return recv
    # point-to-point fallback
    rank = dist.get_rank(group)
    size = dist.get_world_size(group)
    ranks = dist.get_process_group_ranks(group)
    soff = [0]
    roff = [0]
    for a, b in zip(send_counts, recv_counts):
        soff.append(soff[-1] + a)
        roff.append(roff[-1] + b)
    reqs = []
    for peer in range(size):
        if peer == rank:
            recv[roff[peer]:roff[peer + 1]] = send[soff[peer]:soff[peer + 1]]
            continue
        reqs.append(dist.isend(send[soff[peer]:soff[peer + 1]].contiguous(), dst=ranks[peer], group=group))
    bufs = {}
    for peer in range(size):
        if peer == rank:
            continue
        bufs[peer] = send.new_empty(recv_counts[peer])
        reqs.append(dist.irecv(bufs[peer], src=ranks[peer], group=group))
    for r in reqs:
        r.wait()
    for peer, b in bufs.items():
        recv[roff[peer]:roff[peer + 1]] = b
    return recv


def _transpose(x: torch.Tensor, dim0: int, dim1: int, dim1_split_sizes, group):
    """Scatter ``dim0``, gather ``dim1`` across ``group``; returns the redistributed contiguous tensor.

    On the wire every piece keeps the tensor's own axis order: peer j receives this rank's slice ``dim0 in chunk j`` and
    this rank receives from peer j the slice that carries ``dim1`` chunk j.  The send buffer is therefore one gather of the
    chunks (no copy at all when ``dim0`` is the leading axis: the chunks already lie one after the other) and the result is
    one concatenation along ``dim1`` (no copy when ``dim1`` is the leading axis: the received pieces already are the result)."""
    size = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if size == 1:
        return x
    nd = x.dim()
    dim0 %= nd
    dim1 %= nd
    if config.debug:
        _verify("_transpose: error, dim1_split_sizes", x.shape[dim1], list(dim1_split_sizes), group)
    is_complex = x.is_complex()
    xr = torch.view_as_real(x.resolve_conj()) if is_complex else x  # trailing (re, im) axis does not move
    xr = xr.contiguous()
    d0 = compute_split_shapes(x.shape[dim0], size)
    per0 = xr.numel() // x.shape[dim0] if x.shape[dim0] else 0   # elements per index of dim0
    send_counts = [c * per0 for c in d0]
    if dim0 == 0:
        send = xr.reshape(-1)
    else:
        send = torch.cat([p.reshape(-1) for p in torch.split(xr, d0, dim=dim0)])
    # what arrives from peer j: my dim0 chunk, with dim1 of length dim1_split_sizes[j]
    rest = per0 // x.shape[dim1] if x.shape[dim1] else 0         # elements per (dim0 index, dim1 index)
    recv_counts = [d0[rank] * rest * s for s in dim1_split_sizes]
    recv = _exchange(send, send_counts, recv_counts, group)
    shape = list(xr.shape)
    shape[dim0] = d0[rank]
    if dim1 == 0:
        shape[dim1] = sum(dim1_split_sizes)
        out = recv.view(shape)
    else:
        pieces, off = [], 0
        for j, s_ in enumerate(dim1_split_sizes):
            shp = list(shape)
            shp[dim1] = s_
            pieces.append(recv[off:off + recv_counts[j]].view(shp))
            off += recv_counts[j]
        out = torch.cat(pieces, dim=dim1)
    return torch.view_as_complex(out) if is_complex else out


def _pieces_exchange_in(x: torch.Tensor, split_sizes, group, axis: int = -1):
    """First half of a transpose that scatters the LEADING axis and gathers ``axis``, stopped before the concatenation:
    ``x`` (n, ..., local length of axis, ...) contiguous -> (flat real buffer, n_local) where the buffer holds, one after
    the other, the blocks (n_local, ..., split_sizes[j], ...) received from the peers j ("piece-major": every block is a
    contiguous tensor of its own).  No copy on either side."""
    size, rank = dist.get_world_size(group), dist.get_rank(group)
    xr = torch.view_as_real(x.resolve_conj()) if x.is_complex() else x
    xr = xr.contiguous()
    d0 = compute_split_shapes(x.shape[0], size)
    per0 = xr.numel() // x.shape[0]
    other = per0 // x.shape[axis]  # elements per (leading index, index of the gathered axis)
    recv = _exchange(xr.reshape(-1), [c * per0 for c in d0], [d0[rank] * other * s for s in split_sizes], group)
    return recv, d0[rank]


def _pieces_exchange_out(buf: torch.Tensor, n_local: int, n_total: int, rest_shape, axis: int, split_sizes, is_complex: bool, group):
    """Second half of a transpose that scatters ``axis`` and gathers the LEADING axis, started from a piece-major buffer:
    ``buf`` holds the blocks (n_local, *rest_shape) with ``rest_shape[axis] = split_sizes[j]``; block j goes to peer j as it
    lies, and what comes back is (n_total, *rest_shape) with ``rest_shape[axis] = split_sizes[rank]`` as it lies.  No copy
    on either side.  ``axis`` counts inside ``rest_shape`` (the entry there is ignored)."""
    size, rank = dist.get_world_size(group), dist.get_rank(group)
    rest = list(rest_shape)
    axis %= len(rest)
    other = 2 if is_complex else 1
    for i, s in enumerate(rest):
        if i != axis:
            other *= s
    d0 = compute_split_shapes(n_total, size)
    rest[axis] = split_sizes[rank]
    recv = _exchange(buf.reshape(-1), [n_local * other * s for s in split_sizes], [c * other * rest[axis] for c in d0], group)
    if is_complex:
        return torch.view_as_complex(recv.view(n_total, *rest, 2))
    return recv.view(n_total, *rest)


class _Transpose(torch.autograd.Function):
    """The transposes move bytes and never compute, so they run on whatever dtype arrives; ``custom_fwd`` /
    ``custom_bwd`` make the backward exchange run under the autocast state the forward one saw
    (torch_harmonics/distributed/primitives.py:279-311)."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx, x, dims, dim1_split_sizes, which):
        group = azimuth_group() if which == "azimuth" else polar_group()
        active = is_distributed_azimuth() if which == "azimuth" else is_distributed_polar()
        ctx.which, ctx.dims, ctx.active = which, dims, active
        x = x.contiguous()
        if not active:
            return x
        gsize = azimuth_group_size() if which == "azimuth" else polar_group_size()
        ctx.dim0_split_sizes = compute_split_shapes(x.shape[dims[0]], gsize)
        return _transpose(x, dims[0], dims[1], dim1_split_sizes, group)

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, go):
        go = go.contiguous()
        if not ctx.active:
            return go, None, None, None
        group = azimuth_group() if ctx.which == "azimuth" else polar_group()
        gi = _transpose(go, ctx.dims[1], ctx.dims[0], ctx.dim0_split_sizes, group)
        return gi, None, None, None


@torch.compiler.disable()
def distributed_transpose_azimuth(input_, dims_, shapes_):
    """All-to-all transpose across the azimuth group: sharded along ``dims_[1]`` in, sharded along ``dims_[0]`` out.
    ``shapes_`` lists the per-rank lengths along ``dims_[1]``."""
    return _Transpose.apply(input_, dims_, shapes_, "azimuth")


@torch.compiler.disable()
def distributed_transpose_polar(input_, dims_, shapes_):
    """Same across the polar group."""
    return _Transpose.apply(input_, dims_, shapes_, "polar")


def _all_reduce_sum(t: torch.Tensor, group) -> torch.Tensor:
    """Sum over the ranks of ``group`` in a fresh buffer (the caller's tensor is never written); complex tensors travel
    as (re, im) pairs, half precision is summed in float32 (torch_harmonics/distributed/primitives.py:351-369)."""
    if dist.get_world_size(group=group) == 1:
        return t
    dtype = t.dtype
    if t.is_complex():
        buf = torch.view_as_real(t.contiguous().resolve_conj()).clone()
    elif dtype in (torch.float16, torch.bfloat16):
        buf = t.float().contiguous()  # (a conversion: always a fresh buffer)
    else:
        buf = t.contiguous().clone()
    dist.all_reduce(buf, group=group)
    return torch.view_as_complex(buf) if t.is_complex() else buf.to(dtype)


class _Region(torch.autograd.Function):
    """The two conjugate halves of a replicated-versus-partial bookkeeping across one communicator:

    * ``reduce=False`` ("copy to region"): identity forward, all-reduce of the gradient backward - for a value that is
      the same on every rank of the group and feeds rank-local partial computations;
    * ``reduce=True`` ("reduce from region"): all-reduce forward, identity backward - for partial results that are
      summed into a value every rank then holds.

    torch_harmonics/distributed/primitives.py:506-553 and :616-669."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx, x, which, reduce):
        ctx.which, ctx.reduce = which, reduce
        active = is_distributed_azimuth() if which == "azimuth" else is_distributed_polar()
        if reduce and active:
            return _all_reduce_sum(x, azimuth_group() if which == "azimuth" else polar_group())
        return x.view_as(x)

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, g):
        active = is_distributed_azimuth() if ctx.which == "azimuth" else is_distributed_polar()
        if not ctx.reduce and active:
            g = _all_reduce_sum(g, azimuth_group() if ctx.which == "azimuth" else polar_group())
        return g, None, None


@torch.compiler.disable()
def copy_to_polar_region(input_):
    """Identity forward, sum of the gradients over the polar group backward."""
    return _Region.apply(input_, "polar", False)


@torch.compiler.disable()
def copy_to_azimuth_region(input_):
    """Identity forward, sum of the gradients over the azimuth group backward."""
    return _Region.apply(input_, "azimuth", False)


@torch.compiler.disable()
def reduce_from_polar_region(input_):
    """Sum over the polar group forward, identity backward."""
    return _Region.apply(input_, "polar", True)


@torch.compiler.disable()
def reduce_from_azimuth_region(input_):
    """Sum over the azimuth group forward, identity backward."""
    return _Region.apply(input_, "azimuth", True)
