"""Failures injected on the host: a damaged checkpoint, a data source that raises, a peer that stops
beating or leaves. Nothing here touches a GPU."""
import multiprocessing as mp
import time

import pytest
import torch

from eridiffusion_b200.adapters import AdapterConfig
from eridiffusion_b200.data import synthetic_batch
from eridiffusion_b200.models import build_model
from eridiffusion_b200.parallel.health import Heartbeat, RankFailure
from eridiffusion_b200.train.services import ResilientBatches
from eridiffusion_b200.train.trainer import Trainer, TrainerConfig


def _trainer(out):
    torch.manual_seed(0)
    m = build_model("tiny_mmdit", device="cpu", dtype=torch.float32)
    cfg = TrainerConfig(mode="lora", adapter=AdapterConfig(rank=4, alpha=4, dtype=torch.float32), optimizer="adamw",
                        lr=1e-2, seed=3, out_dir=str(out))
    return Trainer(m, cfg)


def test_damaged_checkpoint_falls_back_to_the_previous_one(tmp_path):
    tr = _trainer(tmp_path)
    for i in range(2):
        tr.train_step(synthetic_batch("tiny_mmdit", 1, "cpu", torch.float32, i))
    tr.save_checkpoint()
    good = {n: p.detach().clone() for n, p in tr.model.named_parameters() if p.requires_grad}
    tr.train_step(synthetic_batch("tiny_mmdit", 1, "cpu", torch.float32, 2))
    tr.save_checkpoint()
    newest = sorted(tmp_path.glob("step_*"))[-1]
    f = newest / "lora.safetensors"
    f.write_bytes(f.read_bytes()[: f.stat().st_size // 2])                 # a crash in the middle of the write
    tr2 = _trainer(tmp_path)
    skipped = []
    from eridiffusion_b200.train.checkpoint import load_latest_training_checkpoint
    r = load_latest_training_checkpoint(tr2, tmp_path, on_skip=lambda p, e: skipped.append(p.name))
    assert r is not None and r[0] == 2 and skipped == [newest.name]
    for n, p in tr2.model.named_parameters():
        if p.requires_grad:
            assert torch.equal(p, good[n].bfloat16().float()), n       # adapters are stored as bf16
    (sorted(tmp_path.glob("step_*"))[0] / "meta.json").write_text("{ not json")
    assert load_latest_training_checkpoint(_trainer(tmp_path), tmp_path) is None   # nothing loadable left


class _Flaky:
    def __init__(self, fail_at, n=8):
        self.i, self.fail_at, self.n = 0, set(fail_at), n

    def __iter__(self):
        return self

    def __next__(self):
        self.i += 1
        if self.i > self.n:
            raise StopIteration
        if self.i in self.fail_at:
            raise OSError(f"cannot read sample {self.i}")
        return self.i


def test_data_source_errors_are_skipped_until_they_persist():
    seen = []
    rb = ResilientBatches(_Flaky({2, 5}), on_error=lambda e: seen.append(str(e)))
    assert list(rb) == [1, 3, 4, 6, 7, 8] and rb.skipped == 2 and len(seen) == 2
    with pytest.raises(OSError):
        list(ResilientBatches(_Flaky({2, 3, 4}), max_consecutive=3))


class _Store(dict):
    def set(self, k, v):
        self[k] = v

    def get(self, k):
        return self[k]


def test_heartbeat_logic_with_a_fake_clock():
    now = [0.0]
    s = _Store()
    a = Heartbeat(s, 0, 3, timeout_s=5.0, clock=lambda: now[0], start=False)
    b = Heartbeat(s, 1, 3, timeout_s=5.0, clock=lambda: now[0], start=False)
    assert a.status() == {0: "alive", 1: "alive", 2: "unknown"}
    now[0] = 4.0
    b.beat()
    a.check()                                             # rank 2 has not joined yet, still within the grace time
    now[0] = 6.0
    with pytest.raises(RankFailure) as e:
        a.check()
    assert e.value.dead == [2] and e.value.left == []
    c = Heartbeat(s, 2, 3, timeout_s=5.0, clock=lambda: now[0], start=False)
    a.check()                                             # it joined: all alive
    now[0] = 12.0
    c.beat()
    with pytest.raises(RankFailure) as e:                 # rank 1 stopped beating at t = 4
        a.check()
    assert e.value.dead == [1]
    b.leave()
    with pytest.raises(RankFailure) as e:
        a.check()
    assert e.value.dead == [] and e.value.left == [1]


def _rank(rank, port, q):
    import datetime
    import torch.distributed as dist
    store = dist.TCPStore("127.0.0.1", port, 2, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30),
                          wait_for_workers=False)
    hb = Heartbeat(store, rank, 2, interval_s=0.1, timeout_s=1.0)
    if rank == 1:
        time.sleep(0.5)                                   # two healthy "steps", then the process dies
        import os
        os._exit(0)
    t0 = time.time()
    try:
        while time.time() - t0 < 20:
            hb.check()                                    # between steps, before the next launch
            time.sleep(0.1)
        q.put(("no failure seen", None))
    except RankFailure as e:
        q.put(("failure", (e.dead, round(time.time() - t0, 1))))
    hb.close()


def test_peer_death_is_noticed_on_the_host():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29000 + (int(time.time() * 1000) % 500)
    ps = [ctx.Process(target=_rank, args=(r, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    kind, info = q.get(timeout=60)
    for p in ps:
        p.join(timeout=30)
    assert kind == "failure" and info[0] == [1] and info[1] < 10


def test_run_training_leaves_with_a_checkpoint_when_a_peer_is_gone(tmp_path):
    from eridiffusion_b200.train.services import run_training
    now = [0.0]
    s = _Store()
    me = Heartbeat(s, 0, 2, timeout_s=5.0, clock=lambda: now[0], start=False)
    peer = Heartbeat(s, 1, 2, timeout_s=5.0, clock=lambda: now[0], start=False)
    tr = _trainer(tmp_path)

    def batches():
        i = 0
        while True:
            if i == 2:
                peer.leave()                              # the peer exits cleanly between steps
            yield synthetic_batch("tiny_mmdit", 1, "cpu", torch.float32, i)
            i += 1

    with pytest.raises(RankFailure) as e:
        run_training(tr, batches(), 10, log_every=100, print_fn=lambda *_: None, heartbeat=me)
    assert e.value.left == [1] and tr.step == 3
    assert sorted(p.name for p in tmp_path.glob("step_*")) == ["step_000003"]


def test_8bit_optimizer_state_resharding(tmp_path):
    from eridiffusion_b200.io import safetensors as st
    from eridiffusion_b200.train.checkpoint import reshard_8bit_state
    g = torch.Generator().manual_seed(0)
    nblk = 12                                            # 12 blocks of 256 saved by 2 ranks
    full = {"m_q": torch.randint(-127, 127, (nblk * 256,), generator=g, dtype=torch.int8),
            "v_q": torch.randint(0, 255, (nblk * 256,), generator=g, dtype=torch.uint8),
            "m_absmax": torch.rand(nblk, generator=g), "v_absmax": torch.rand(nblk, generator=g)}
    files = []
    for r in range(2):
        sl, bl = slice(r * 6 * 256, (r + 1) * 6 * 256), slice(r * 6, (r + 1) * 6)
        f = tmp_path / f"optimizer.rank{r}.safetensors"
        st.save_file({"optimizer.m_q": full["m_q"][sl], "optimizer.v_q": full["v_q"][sl],
                      "optimizer.m_absmax": full["m_absmax"][bl], "optimizer.v_absmax": full["v_absmax"][bl]}, f)
        files.append(f)
    one = reshard_8bit_state(files, 0, 1, nblk * 256)
    assert all(torch.equal(one[k], full[k]) for k in full)
    # 3 ranks: 4 blocks each
    for r in range(3):
        p = reshard_8bit_state(files, r, 3, 4 * 256)
        assert torch.equal(p["m_q"], full["m_q"][r * 1024:(r + 1) * 1024])
        assert torch.equal(p["v_absmax"], full["v_absmax"][r * 4:(r + 1) * 4])
    # 8 ranks need 16 blocks (2 per rank): the tail is zero padding
    last = reshard_8bit_state(files, 7, 8, 2 * 256)
    assert last["m_q"].abs().sum() == 0 and last["v_absmax"].sum() == 0 and last["m_q"].numel() == 512
    p5 = reshard_8bit_state(files, 5, 8, 2 * 256)
    assert torch.equal(p5["v_q"], full["v_q"][10 * 256:12 * 256])


def test_resumed_run_draws_the_same_timesteps_as_an_uninterrupted_one(tmp_path):
    """The timestep generator's state travels with the checkpoint: a run resumed at step k continues
    the stream instead of replaying the draws of step 0."""
    drawn = {}

    def spy(tr, tag):
        orig = tr.objective.sample_t

        def wrapped(n, gen=None, device="cpu"):
            t = orig(n, gen, device)
            drawn.setdefault(tag, []).append(t.clone())
            return t
        tr.objective.sample_t = wrapped

    full = _trainer(tmp_path / "a")
    spy(full, "full")
    for i in range(5):
        full.train_step(synthetic_batch("tiny_mmdit", 1, "cpu", torch.float32, i))
    first = _trainer(tmp_path / "b")
    spy(first, "first")
    for i in range(3):
        first.train_step(synthetic_batch("tiny_mmdit", 1, "cpu", torch.float32, i))
    first.save_checkpoint()
    resumed = _trainer(tmp_path / "b")
    assert resumed.load_latest_checkpoint() == (3, 3)
    spy(resumed, "resumed")
    for i in range(3, 5):
        resumed.train_step(synthetic_batch("tiny_mmdit", 1, "cpu", torch.float32, i))
    got = drawn["first"] + drawn["resumed"]
    assert len(got) == 5 and all(torch.equal(a, b) for a, b in zip(got, drawn["full"]))
    assert not torch.equal(drawn["resumed"][0], drawn["full"][0])      # not a replay from the start


def _ckpt_worker(rank, world, port, root, q):
    import os
    os.environ.update(WORLD_SIZE=str(world), RANK=str(rank), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch
    import torch.distributed as dist
    from pathlib import Path
    from eridiffusion_b200.parallel.dist import GradSync, init_from_env
    from eridiffusion_b200.train.checkpoint import load_latest_training_checkpoint
    torch.set_num_threads(2)
    init_from_env("gloo", timeout_s=120)
    root = Path(root)

    def mk():
        torch.manual_seed(0)
        m = build_model("tiny_mmdit", device="cpu", dtype=torch.float32)
        cfg = TrainerConfig(mode="lora", adapter=AdapterConfig(rank=4, alpha=4, dtype=torch.float32),
                            optimizer="adamw8bit", lr=1e-2, seed=3, out_dir=str(root), stochastic_rounding=False)
        return Trainer(m, cfg, grad_sync=GradSync("zero1"))

    tr = mk()
    for i in range(2):
        tr.train_step(synthetic_batch("tiny_mmdit", 1, "cpu", torch.float32, 10 * i + rank))
    tr.save_checkpoint()
    tr.train_step(synthetic_batch("tiny_mmdit", 1, "cpu", torch.float32, 20 + rank))
    tr.save_checkpoint()
    dist.barrier()
    newest = sorted(root.glob("step_*"))[-1]
    # every rank wrote its shard before meta.json appeared
    assert all((newest / f"optimizer.rank{r}.safetensors").exists() for r in range(world))
    if rank == 1:
        f = newest / "optimizer.rank1.safetensors"                    # damage ONE rank's shard only
        f.write_bytes(f.read_bytes()[: f.stat().st_size // 2])
    dist.barrier()
    tr2 = mk()
    skipped = []
    res = load_latest_training_checkpoint(tr2, root, on_skip=lambda p, e: skipped.append(p.name))
    q.put((rank, res, skipped, tr2.step))
    dist.barrier()
    dist.destroy_process_group()


def test_one_damaged_shard_makes_every_rank_fall_back_together(tmp_path):
    """Two gloo ranks with sharded 8-bit optimizer state: a truncated shard of rank 1 must send BOTH
    ranks to the previous checkpoint, so that they resume at the same step."""
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_ckpt_worker, args=(r, 2, port, str(tmp_path), q)) for r in range(2)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=240) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, res0, skip0, step0), (r1, res1, skip1, step1) = out
    assert res0 == res1 == (2, 3) and step0 == step1 == 2
    assert skip0 == skip1 == ["step_000003"]
