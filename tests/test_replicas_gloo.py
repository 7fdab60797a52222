"""CPU: the multi-GPU path is independent replicas that shard the global batch; what the ranks share is the timing
reduction (max over ranks of the time, sum over ranks of the work) and the rule that only rank 0 reports.  Exercised with
two gloo ranks."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, json
sys.path.insert(0, os.environ["REPO"])
import torch.distributed as dist
import bench
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
ms = [100.0 + 50.0 * rank, 7.0 - rank, 3.0]          # rank 1 is slower on the first, faster on the second
mx = bench.max_over_ranks(ms, world)
sm = bench.sum_over_ranks([1.0 + rank, 10.0], world)
dist.barrier()
if rank == 0:
    cfg = bench.config_for(world)
    print(json.dumps({"mx": mx, "sm": sm, "per": cfg["per_gpu_batch"], "value": bench.sharded_throughput(cfg["global_batch"], 10, mx[0])}))
dist.destroy_process_group()
'''


def test_two_rank_timing_reduction(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, REPO=ROOT)
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                          "--master-port", "29571", str(script)], env=env, capture_output=True, text=True, timeout=240)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1                       # only rank 0 reports
    got = json.loads(lines[0])
    assert got["mx"] == [150.0, 7.0, 3.0]        # element-wise max over the two ranks
    assert got["sm"] == [3.0, 20.0]
    assert got["per"] == 32                      # the global batch of 64 is sharded, not replicated
    assert abs(got["value"] - 64 * 10 * 1000.0 / 150.0) < 1e-9


def test_reference_arm_runs_on_rank0_only():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
                         env=env, capture_output=True, text=True, timeout=240)
    assert out.returncode == 0 and out.stdout.strip() == ""   # other ranks exit 0 without work


def test_reference_arm_reports_the_same_config_as_the_gpu_arm():
    """The host arm's line carries the configuration dict of the GPU arm (the driver compares them) and a per-image
    throughput that is measured, not extrapolated."""
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][0])
    sys.path.insert(0, ROOT)
    import bench
    assert line["impl"] == "reference" and line["config"] == bench.config_for(1)
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert abs(line["value"] * line["ms_per_step"] / 1000.0 - 1.0) < 1e-6   # one image per step: value = 1 / step time
