"""GEMM operand modes that carry the fused-communication paths: MN-major B, gathers executed by
copy CTAs inside the launch (peers emulated by local buffers on one GPU), peer scatter epilogue."""
import pytest
import torch

from eridiffusion_b200.ops import functional as F
from eridiffusion_b200.parallel.gather_gemm import GatherPlan

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*s, seed=0, scale=1.0):
    g = torch.Generator(device=DEV).manual_seed(seed + sum(s))
    return (torch.randn(*s, device=DEV, generator=g) * scale).bfloat16()


def close(a, b, atol):
    err = (a.float() - b.float()).abs().max().item()
    assert err <= atol + 0.02 * b.float().abs().max().item(), err


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (512, 1024, 320), (384, 192, 256)])
def test_b_mn(M, N, K):
    a, bt = rnd(M, K), rnd(K, N, seed=1)
    out = F.gemm_native(a, bt, b_mn=True)
    assert F.gemm_error_check() == 0
    close(out, a.float() @ bt.float(), 0.05)


@pytest.mark.parametrize("rank", [0, 2])
def test_gather_rows_forward(rank):
    W, M, N, K = 4, 512, 1024, 512
    x = rnd(M, K)
    shards = [rnd(N // W, K, seed=10 + p, scale=K ** -0.5) for p in range(W)]
    landing = torch.full((N, K), float("nan"), device=DEV, dtype=torch.bfloat16)
    plan = GatherPlan.rows(rank, W, [s.data_ptr() for s in shards], landing, n_copy=4)
    out = F.gemm_native(x, landing, gather=plan.launch_args())
    assert F.gemm_error_check() == 0
    w = torch.cat(shards, 0)
    per = N // W
    for p in range(W):                       # the own slab may be read in place and never land
        if p != rank:
            assert torch.equal(landing[p * per:(p + 1) * per], shards[p])
    close(out, x.float() @ w.float().t(), 0.05)


@pytest.mark.parametrize("join_round", [1, 2, 50])
def test_gather_copy_clusters_join_the_tile_loop(join_round):
    """Copy clusters that take tiles once their slabs have landed (from a given round of the persistent
    schedule on; a round beyond the last leaves them idle): same result, every tile computed once."""
    W, rank, M, N, K = 4, 1, 4096, 8192, 256          # 512 pair tiles: several rounds on 74 clusters
    x = rnd(M, K)
    shards = [rnd(N // W, K, seed=10 + p, scale=K ** -0.5) for p in range(W)]
    landing = torch.full((N, K), float("nan"), device=DEV, dtype=torch.bfloat16)
    plan = GatherPlan.rows(rank, W, [s.data_ptr() for s in shards], landing, n_copy=8)
    out = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    c0 = F.N.require().eri_gemm2_gather_count()
    F.gemm_native(x, landing, out=out, gather=dict(plan.launch_args(), join_round=join_round))
    assert F.gemm_error_check() == 0 and F.N.require().eri_gemm2_gather_count() == c0 + 1
    close(out, x.float() @ torch.cat(shards, 0).float().t(), 0.05)


@pytest.mark.parametrize("rank", [1, 3])
def test_gather_rows_along_k_for_input_grad(rank):
    W, M, N, K = 4, 384, 1024, 512          # dX[M, K] = dY[M, N] @ W[N, K]
    dy = rnd(M, N)
    shards = [rnd(N // W, K, seed=20 + p, scale=N ** -0.5) for p in range(W)]
    landing = torch.full((N, K), float("nan"), device=DEV, dtype=torch.bfloat16)
    plan = GatherPlan.rows(rank, W, [s.data_ptr() for s in shards], landing, along_k=True, n_copy=4)
    out = F.gemm_native(dy, landing, b_mn=True, gather=plan.launch_args())
    assert F.gemm_error_check() == 0
    w = torch.cat(shards, 0)
    close(out, dy.float() @ w.float(), 0.05)


def test_gather_cols_reverse_all_to_all():
    W, L, Cc, N = 4, 256, 128, 512            # out-proj input [L, W*Cc] from W peers
    rank = 1
    srcs = [rnd(W * L, Cc, seed=30 + p) for p in range(W)]       # peer p's attention output
    wo = rnd(N, W * Cc, seed=50, scale=(W * Cc) ** -0.5)
    landing = torch.full((L, W * Cc), float("nan"), device=DEV, dtype=torch.bfloat16)
    plan = GatherPlan.cols(rank, W, [s.data_ptr() for s in srcs], rank * L, Cc * 2, landing, n_copy=4)
    out = F.gemm_native(landing, wo, gather=plan.launch_args())
    assert F.gemm_error_check() == 0
    a = torch.cat([s[rank * L:(rank + 1) * L] for s in srcs], 1)
    for p in range(W):                       # the own column block may be read in place and never land
        if p != rank:
            assert torch.equal(landing[:, p * Cc:(p + 1) * Cc], a[:, p * Cc:(p + 1) * Cc])
    close(out, a.float() @ wo.float().t(), 0.05)


def test_scatter_epilogue_routes_head_groups():
    W, rank, B, Ll, H, Dh, K = 2, 1, 2, 128, 4, 64, 256
    part = H * Dh                  # 256 columns per q / k / v part
    group = part // W              # 128 columns per rank
    x = rnd(B * Ll, K)
    wqkv = rnd(3 * part, K, seed=1, scale=K ** -0.5)
    bias = rnd(3 * part, seed=2)
    dests = [torch.zeros(B * W * Ll, 3 * group, device=DEV, dtype=torch.bfloat16) for _ in range(W)]
    F.gemm_native(x, wqkv, bias=bias, out=dests[0],
                  scatter=dict(world=W, rank=rank, part_cols=part, group_cols=group, local_rows=Ll,
                               ptrs=[d.data_ptr() for d in dests]))
    assert F.gemm_error_check() == 0
    y = (x.float() @ wqkv.float().t() + bias.float()).view(B, Ll, 3, W, group)
    for d in range(W):
        got = dests[d].view(B, W, Ll, 3, group)
        close(got[:, rank], y[:, :, :, d], 0.05)
        assert got[:, 1 - rank].abs().max().item() == 0.0


@pytest.mark.parametrize("N,K", [(9216, 256), (3072, 512)])
def test_gather_rows_unaligned_slabs_stay_on_the_pair_kernel(N, K):
    """Eight ranks with slabs of 1152 / 384 rows (not multiples of the 256-column pair tile): every
    emulated rank must run on the two-CTA kernel, forward and input-gradient direction."""
    W, M = 8, 512
    lib = F.N.require()
    x = rnd(M, K)
    dy = rnd(M, N, seed=3)
    shards = [rnd(N // W, K, seed=10 + p, scale=K ** -0.5) for p in range(W)]
    w = torch.cat(shards, 0)
    ref_y = x.float() @ w.float().t()
    ref_dx = dy.float() @ w.float()
    for rank in range(W):
        landing = torch.full((N, K), float("nan"), device=DEV, dtype=torch.bfloat16)
        plan = GatherPlan.rows(rank, W, [s.data_ptr() for s in shards], landing, n_copy=4)
        c0 = lib.eri_gemm2_gather_count()
        out = F.gemm_native(x, landing, gather=plan.launch_args())
        assert lib.eri_gemm2_gather_count() == c0 + 1, f"rank {rank} fell back to the one-CTA kernel"
        assert F.gemm_error_check() == 0
        close(out, ref_y, 0.05)
        landing.fill_(float("nan"))
        plan = GatherPlan.rows(rank, W, [s.data_ptr() for s in shards], landing, along_k=True, n_copy=4)
        c0 = lib.eri_gemm2_gather_count()
        dx = F.gemm_native(dy, landing, b_mn=True, gather=plan.launch_args())
        assert lib.eri_gemm2_gather_count() == c0 + 1, f"rank {rank} (dX) fell back to the one-CTA kernel"
        assert F.gemm_error_check() == 0
        close(dx, ref_dx, 0.05 * (N / 1024) ** 0.5)


@pytest.mark.parametrize("pair", [True, False])
def test_scatter_epilogue_pair_tiles_and_row_squares(pair, monkeypatch):
    """Head groups of 512 columns (whole 256-column pair tiles): the scatter epilogue of the two-CTA
    kernel against the one-CTA kernel and the fp32 statement, with the QK-norm row sums."""
    monkeypatch.setattr(F, "_SCATTER_PAIR", pair)
    W, rank, B, Ll, H, Dh, K = 2, 1, 1, 384, 8, 128, 320
    part = H * Dh                  # 1024 columns per q / k / v part
    group = part // W              # 512 columns per rank
    x = rnd(B * Ll, K)
    wqkv = rnd(3 * part, K, seed=1, scale=K ** -0.5)
    bias = rnd(3 * part, seed=2)
    dests = [torch.zeros(B * W * Ll, 3 * group, device=DEV, dtype=torch.bfloat16) for _ in range(W)]
    rowsq = torch.zeros(2, B * Ll, device=DEV, dtype=torch.float32)
    F.gemm_native(x, wqkv, bias=bias, out=dests[0],
                  scatter=dict(world=W, rank=rank, part_cols=part, group_cols=group, local_rows=Ll,
                               ptrs=[d.data_ptr() for d in dests], rowsq=rowsq))
    assert F.gemm_error_check() == 0
    yf = x.float() @ wqkv.float().t() + bias.float()
    y = yf.view(B, Ll, 3, W, group)
    for d in range(W):
        got = dests[d].view(B, W, Ll, 3, group)
        close(got[:, rank], y[:, :, :, d], 0.05)
        assert got[:, 1 - rank].abs().max().item() == 0.0
    want_sq = yf.view(B * Ll, 3, part)[:, :2].pow(2).sum(-1).t()
    assert torch.allclose(rowsq, want_sq, rtol=2e-2, atol=1e-2)


@pytest.mark.parametrize("rank", [0, 2])
def test_row_slab_scatter_is_the_weight_gradient_reduce_scatter(rank):
    """dW = dY^T X whose epilogue pushes row slab d of the result into slot `rank` of rank d's receive
    buffer (peers emulated by local buffers); the owner then adds the slots."""
    W, T, N, K = 4, 640, 1024, 512
    per = N // W
    dy, x = rnd(T, N, scale=0.5), rnd(T, K, seed=1)
    recv = [torch.zeros(W, per, K, device=DEV, dtype=torch.bfloat16) for _ in range(W)]
    F.gemm_native(dy, x, a_mn=True, b_mn=True, out=recv[0].view(N, K),
                  scatter=dict(world=W, rank=rank, mode=1, local_rows=per, part_cols=0, group_cols=0,
                               ptrs=[r.data_ptr() for r in recv]))
    assert F.gemm_error_check() == 0
    ref = dy.float().t() @ x.float()
    for d in range(W):
        close(recv[d][rank], ref[d * per:(d + 1) * per], 0.05 * (T / 128) ** 0.5)
        others = [s for s in range(W) if s != rank]
        assert recv[d][others].abs().max().item() == 0.0
    # the owner's reduction over the slots (mean over ranks), here with every slot filled differently
    slots = torch.stack([rnd(per, K, seed=40 + s) for s in range(W)])
    out = torch.empty(per, K, device=DEV, dtype=torch.bfloat16)
    lib = F.N.require()
    F.N.check(lib.eri_slot_reduce(slots.data_ptr(), out.data_ptr(), W, per * K, 1.0 / W, 0, F.N.stream_ptr()), "slot_reduce")
    close(out, slots.float().mean(0), 0.02)
    acc = out.clone()
    F.N.check(lib.eri_slot_reduce(slots.data_ptr(), acc.data_ptr(), W, per * K, 1.0 / W, 1, F.N.stream_ptr()), "slot_reduce")
    close(acc, 2 * slots.float().mean(0), 0.04)
