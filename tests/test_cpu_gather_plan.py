"""Host-side planning of the gather-fused GEMM: job lists, landing counters and the in-place local
slab, built on CPU tensors with made-up peer addresses (nothing is launched)."""
import torch

from eridiffusion_b200.parallel.gather_gemm import GatherOrder, GatherPlan


def _ptrs(world, stride):
    return [0x10000000 + p * stride for p in range(world)]


def test_rows_plan_counters_and_local_slab():
    W, rank, Nn, K = 4, 2, 2048, 512
    landing = torch.empty(Nn, K, dtype=torch.bfloat16)
    per = Nn // W
    pl = GatherPlan.rows(rank, W, _ptrs(W, per * K * 2), landing, n_copy=8, rows_per_job=64, flag_rows=256)
    # one counter per 256 rows plus the counter that every job bumps ("everything has landed")
    assert len(pl.flags) == Nn // 256 + 1 and pl.kw == dict(b_flag_rows=256, rot_n_rows=rank * per)
    # every 256-row counter expects its four 64-row jobs; without the local slab its counters expect none
    assert pl.targets == [4] * 8 + [32]
    own = [f for f in range(8) if rank * per <= f * 256 < (rank + 1) * per]
    assert [pl.targets_nl[f] for f in own] == [0, 0] and pl.targets_nl[-1] == 4 * 6 == sum(pl.targets_nl[:-1])
    assert len(pl.jobs) == W * per // 64 and len(pl.jobs_nl) == (W - 1) * per // 64
    assert pl.bytes_from_peers() == (W - 1) * per * K * 2
    assert pl.local == dict(ptr=_ptrs(W, per * K * 2)[rank], ld=K, mode=1, lo=rank * per, hi=(rank + 1) * per)
    # the own slab's jobs come first in the full list (tiles start there), peers are interleaved after it
    first = pl.jobs[0]
    assert first.src == pl.local["ptr"] and first.flag == rank * per // 256
    dst0 = landing.data_ptr() + rank * per * K * 2
    assert first.dst == dst0 and first.rows == 64 and first.row_bytes == K * 2
    args = pl.launch_args()
    assert args["n_jobs"] == len(pl.jobs) and args["local"]["n_jobs"] == len(pl.jobs_nl) and args["local"]["mode"] == 1


def test_rows_plan_along_k_has_one_counter_per_slab():
    W, rank, Nn, K = 8, 5, 9216, 136               # K_in not a multiple of 256: counters per range of the reduction
    landing = torch.empty(Nn, K, dtype=torch.bfloat16)
    per = Nn // W                                  # 1152 rows: not a multiple of 256 -> 128-row counters
    pl = GatherPlan.rows(rank, W, _ptrs(W, per * K * 2), landing, along_k=True, n_copy=16)
    # along the reduction dimension every tile walks all slabs: one counter per slab (a counter costs
    # the producer a global load in the middle of its K loop), plus the "everything has landed" counter
    assert len(pl.flags) == W + 1 and pl.kw == dict(a_flag_cols=per, rot_k_cols=rank * per)
    assert pl.targets[:-1] == [per // 64] * W      # eighteen 64-row jobs per slab
    assert pl.targets[-1] == len(pl.jobs) and pl.targets_nl[-1] == len(pl.jobs_nl)
    assert pl.targets_nl[rank] == 0 and pl.local["mode"] == 2


def test_rows_plan_rotation_is_a_whole_pair_tile_on_every_rank():
    # the two shapes whose slabs are not multiples of 256 rows at 8 ranks
    for Nn in (9216, 3072):
        W, K = 8, 128
        per = Nn // W
        landing = torch.empty(Nn, K, dtype=torch.bfloat16)
        for rank in range(W):
            pl = GatherPlan.rows(rank, W, _ptrs(W, per * K * 2), landing, n_copy=16)
            assert pl.kw["b_flag_rows"] == 128 and pl.kw["rot_n_rows"] % 256 == 0
            # the tile order starts INSIDE this rank's own slab (rounded up to the next pair tile), never
            # in the previous rank's slab, which the copy CTAs fill last
            assert rank * per <= pl.kw["rot_n_rows"] < rank * per + 256 and pl.kw["rot_n_rows"] < (rank + 1) * per
            # copy jobs: slab after slab in ring order from the own slab
            owners = [j.flag * 128 // per for j in pl.jobs]
            assert owners == sorted(owners, key=lambda p: (p - rank) % W)
            assert pl.local["lo"] % 128 == 0 and pl.local["hi"] % 128 == 0
            # every counter is bumped by exactly the jobs that cover its rows
            rows_per_flag = [0] * (len(pl.flags) - 1)
            for j in pl.jobs:
                rows_per_flag[j.flag] += j.rows
            assert rows_per_flag == [128] * (Nn // 128)
            pk = GatherPlan.rows(rank, W, _ptrs(W, per * K * 2), landing, along_k=True, n_copy=16)
            assert pk.kw["rot_k_cols"] % 64 == 0 and pk.kw["a_flag_cols"] == per


def test_cols_plan_row_groups_and_local_block():
    W, rank, L, Cc = 4, 1, 384, 128
    landing = torch.empty(L, W * Cc, dtype=torch.bfloat16)
    src = _ptrs(W, W * L * Cc * 2)
    pl = GatherPlan.cols(rank, W, src, rank * L, Cc * 2, landing, n_copy=4, rows_per_job=128)
    groups = L // 128
    assert len(pl.flags) == W * groups + 1 and pl.targets == [1] * (W * groups) + [W * groups]
    assert pl.kw == dict(a_flag_cols=Cc, rot_k_cols=rank * Cc, a_flag_rows=128)
    assert [pl.targets_nl[rank * groups + g] for g in range(groups)] == [0] * groups
    assert pl.local["mode"] == 3 and pl.local["ptr"] == src[rank] + rank * L * Cc * 2 and pl.local["ld"] == Cc
    j = pl.jobs_nl[0]
    assert j.row_bytes == Cc * 2 and j.src_stride == Cc * 2 and j.dst_stride == W * Cc * 2


def test_gather_order_records_a_step_and_follows_it():
    o = GatherOrder()
    o.begin()
    step = ["qkv", "proj", "mlp0", "mlp2", "mlp2'", "mlp0'", "proj'", "qkv'"]
    assert [o.advance(k) for k in step] == [None] * 8          # first step: nothing recorded yet
    o.begin()
    # second step: every gather names its successor, the last one has none (the shards change after it)
    assert [o.advance(k) for k in step] == step[1:] + [None]
    # a step that leaves the order (a validation forward in between) stops following at once ...
    o.begin()
    got = [o.advance(k) for k in ["qkv", "proj", "other", "mlp0"]]
    assert got == ["proj", "mlp0", None, None]
    # ... and what it did becomes the next expectation
    o.begin()
    assert [o.advance(k) for k in ["qkv", "proj", "other", "mlp0"]] == ["proj", "other", "mlp0", None]
    # a step longer than the recorded one: no successor beyond the record, no error
    o.begin()
    assert [o.advance(k) for k in ["qkv", "proj", "other", "mlp0", "extra"]] == ["proj", "other", "mlp0", None, None]
    # switched off: records, never names a successor
    o.begin(enabled=False)
    assert [o.advance(k) for k in ["qkv", "proj"]] == [None, None]
    # an empty step keeps the last recorded order
    o.begin()
    o.begin()
    assert o.advance("qkv") == "proj"
