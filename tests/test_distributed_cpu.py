"""CPU checks of the distributed host logic with two gloo ranks: split helpers, the all-to-all transposes
(exact after gathering, forward and backward, even and uneven splits, real and complex), the process-grid
registry.  Mirrors torch-harmonics tests/test_distributed_primitives.py:71-220."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, which):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import torch_harmonics_b200.distributed as thd

    group = dist.new_group(list(range(world)))
    if which == "azimuth":
        thd.init(None, group)
        tr = thd.distributed_transpose_azimuth
        assert thd.azimuth_group_size() == world and thd.polar_group_size() == 1 and thd.azimuth_group_rank() == rank
    else:
        thd.init(group, None)
        tr = thd.distributed_transpose_polar
        assert thd.polar_group_size() == world and thd.azimuth_group_size() == 1 and thd.polar_group_rank() == rank
    assert thd.is_initialized()
    thd.config.debug = True  # exercises the shape-verification all-gathers too

    for shape, dims, dtype in (((5, 3, 7, 9), (-3, -1), torch.float32), ((4, 6, 33, 65), (1, 2), torch.float64), ((3, 8, 5), (0, 2), torch.complex64), ((2, 2, 4), (-1, -3), torch.float32),
                               ((3, 4, 2, 5, 6), (-4, -1), torch.float32), ((3, 4, 2, 5, 6), (-2, -4), torch.complex64)):
        g = torch.Generator().manual_seed(1)
        if dtype.is_complex:
            full = torch.complex(torch.randn(shape, generator=g), torch.randn(shape, generator=g))
        else:
            full = torch.randn(shape, generator=g, dtype=dtype)
        d0, d1 = dims[0] % len(shape), dims[1] % len(shape)
        s1 = thd.compute_split_shapes(shape[d1], world)
        s0 = thd.compute_split_shapes(shape[d0], world)
        local = thd.split_tensor_along_dim(full, d1, world)[rank].clone().requires_grad_(not dtype.is_complex)
        out = tr(local, dims, s1)
        expect = thd.split_tensor_along_dim(full, d0, world)[rank]
        assert out.shape == expect.shape and torch.equal(out.detach(), expect), (shape, dims)
        # the reverse transpose restores the tile, and autograd's backward is that reverse transpose
        back = tr(out.detach(), (dims[1], dims[0]), s0)
        assert torch.equal(back, local.detach())
        if not dtype.is_complex:
            out.backward(expect.clone())
            assert torch.equal(local.grad, local.detach())

    thd.config.debug = False

    # copy-to-region / reduce-from-region: conjugate pairs (identity one way, sum over the group the other way); the group
    # that is not distributed leaves values and gradients alone (torch-harmonics tests/test_distributed_primitives.py)
    copy_here, reduce_here = (thd.copy_to_azimuth_region, thd.reduce_from_azimuth_region) if which == "azimuth" else (thd.copy_to_polar_region, thd.reduce_from_polar_region)
    copy_other, reduce_other = (thd.copy_to_polar_region, thd.reduce_from_polar_region) if which == "azimuth" else (thd.copy_to_azimuth_region, thd.reduce_from_azimuth_region)
    for dtype in (torch.float32, torch.complex64, torch.bfloat16):
        base = torch.arange(6, dtype=torch.float32).reshape(2, 3) + 1
        v = (base * (rank + 1)).to(dtype)
        if dtype.is_complex:
            v = v * (1 + 2j)
        total = sum((base * (r + 1)) for r in range(world)).to(dtype) * ((1 + 2j) if dtype.is_complex else 1)
        a = v.clone().requires_grad_(True)
        out = reduce_here(a)
        assert torch.equal(out.detach(), total) and torch.equal(a.detach(), v)  # the input is not written
        out.backward(torch.ones_like(out) * (rank + 2))
        assert torch.equal(a.grad, torch.ones_like(v) * (rank + 2))
        b = v.clone().requires_grad_(True)
        out = copy_here(b)
        assert torch.equal(out.detach(), v)
        out.backward(v.detach().clone())
        assert torch.equal(b.grad, total)
        c = v.clone().requires_grad_(True)
        out = reduce_other(copy_other(c))
        out.backward(torch.ones_like(out))
        assert torch.equal(out.detach(), v) and torch.equal(c.grad, torch.ones_like(v))

    # the distributed quadrature holds this rank's tile of the serial module's weights
    import torch_harmonics_b200 as th

    for grid, shape in (("equiangular", (33, 64)), ("legendre-gauss", (32, 64)), ("lobatto", (17, 30))):
        for normalize in (False, True):
            qs = th.QuadratureS2(shape, grid=grid, normalize=normalize)
            qd = thd.DistributedQuadratureS2(shape, grid=grid, normalize=normalize)
            full = qs.quad_weight
            tile = thd.split_tensor_along_dim(full, -1 if which == "azimuth" else -2, world)[rank]
            assert qd.quad_weight.shape == tile.shape and torch.equal(qd.quad_weight, tile)
    with pytest.raises(ValueError):
        thd.DistributedQuadratureS2((8, 16), grid="nonsense")
    with pytest.raises(RuntimeError):
        thd.DistributedQuadratureS2((8, 16))(torch.zeros(1, 8, 16))  # no CPU path

    with pytest.raises(RuntimeError):
        thd.compute_split_shapes(1, 2)
    thd.finalize()
    assert not thd.is_initialized() and thd.polar_group_size() == 1
    dist.destroy_process_group()


def _pieces_worker(rank, world, port):
    """The two halves of a copy-free transpose (piece-major buffers) against slices of the full tensor."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import torch_harmonics_b200.distributed as thd
    from torch_harmonics_b200.distributed.primitives import _pieces_exchange_in, _pieces_exchange_out

    group = dist.new_group(list(range(world)))
    for shape, axis, dtype in (((9, 5, 14), -1, torch.float32), ((world, 3, 10), -1, torch.complex64), ((7, 2, 11, 6), -2, torch.complex64), ((6, 13, 4), -2, torch.float32)):
        g = torch.Generator().manual_seed(3)
        full_in = torch.randn(shape, generator=g, dtype=torch.float64).to(torch.float32)
        full_out = torch.randn(shape, generator=g, dtype=torch.float64).to(torch.float32)
        if dtype.is_complex:
            full_in = torch.complex(full_in, torch.randn(shape, generator=g))
            full_out = torch.complex(full_out, torch.randn(shape, generator=g))
        ax = axis % len(shape)
        n_splits = thd.compute_split_shapes(shape[0], world)
        a_splits = thd.compute_split_shapes(shape[ax], world)
        n0 = sum(n_splits[:rank])
        mine = slice(n0, n0 + n_splits[rank])

        def flat(t):
            return (torch.view_as_real(t.contiguous()) if t.is_complex() else t.contiguous()).reshape(-1)

        # in: every rank holds all fields and its chunk of `axis`; afterwards its fields, the axis in pieces
        x_local = thd.split_tensor_along_dim(full_in, ax, world)[rank].contiguous()
        buf, n_loc = _pieces_exchange_in(x_local, a_splits, group, axis=axis)
        expect = torch.cat([flat(c) for c in torch.split(full_in[mine], a_splits, dim=ax)])
        assert n_loc == n_splits[rank] and torch.equal(buf, expect), (shape, axis)
        # out: every rank holds its fields with the axis in pieces; afterwards all fields and its chunk of the axis
        pieces = torch.cat([flat(c) for c in torch.split(full_out[mine], a_splits, dim=ax)])
        out = _pieces_exchange_out(pieces, n_loc, shape[0], shape[1:], ax - 1, a_splits, dtype.is_complex, group)
        assert torch.equal(out, thd.split_tensor_along_dim(full_out, ax, world)[rank]), (shape, axis)
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3, 4])
def test_piece_major_exchanges(world):
    mp.spawn(_pieces_worker, args=(world, _free_port()), nprocs=world, join=True)


@pytest.mark.parametrize("which", ["azimuth", "polar"])
def test_transposes_two_ranks(which):
    mp.spawn(_worker, args=(2, _free_port(), which), nprocs=2, join=True)


def test_split_helpers():
    import torch_harmonics_b200.distributed as thd

    assert thd.compute_split_shapes(256, 4) == [64] * 4
    assert thd.compute_split_shapes(128, 3) == [43, 43, 42]
    assert thd.compute_split_shapes(10, 4) == [3, 3, 2, 2]
    assert thd.compute_split_shapes(721, 2) == [361, 360]
    for size in (7, 33, 720):
        for n in (1, 2, 3, 4, 7):
            s = thd.compute_split_shapes(size, n)
            assert sum(s) == size and max(s) - min(s) <= 1 and sorted(s, reverse=True) == s
    x = torch.arange(2 * 3 * 4 * 5, dtype=torch.float32).reshape(2, 3, 4, 5)
    y, lead, n = thd.flatten_and_pad_leading_dims(x, 8)
    assert y.shape == (8, 4, 5) and lead == (2, 3) and n == 6 and torch.all(y[6:] == 0)
    assert torch.equal(thd.unpad_and_unflatten_leading_dims(y, lead, n), x)
    y, lead, n = thd.flatten_and_pad_leading_dims(x, 4)
    assert y.shape == (6, 4, 5)
    xv = torch.zeros(3, 2, 4, 5)
    y, lead, n = thd.flatten_and_pad_leading_dims(xv, 4, num_trailing_dims=3)
    assert y.shape == (4, 2, 4, 5) and n == 3
    # no groups registered: transposes are the identity
    assert torch.equal(thd.distributed_transpose_azimuth(x, (0, 1), [3]), x)
