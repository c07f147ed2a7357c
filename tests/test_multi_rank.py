"""The multi-GPU launch path of bench.py on CPU: two gloo ranks through torch.distributed.run,
barrier + max-over-ranks timing + whole-job aggregation (no GPU, fake per-rank timings)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_two_rank_launch_aggregates_the_slowest_rank():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "4", "--warmup", "1", "--dry-run"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1                      # rank 0 alone prints
    rec = json.loads(lines[0])
    assert rec["n_gpus"] == 2 and rec["scaling"] == "weak"
    # fake timings: rank r takes 10 * steps * (1 + 0.1 r) ms -> the slower rank (1) sets the time
    assert abs(rec["ms_per_step"] - 11.0) < 1e-6
    assert abs(rec["value"] - 32 * 4 * 2 / (44.0e-3)) < 1e-3
    # the two splits of the multi-GPU legs: global batch 32 cut in rank order; one network per half of the ranks
    assert rec["strong"]["shards"] == [[0, 16], [16, 32]]
    assert rec["by_model"]["assignment"] == [["resnet50", 16], ["vgg16", 16]]
    assert rec["strong"]["graphs_in_rotation"] == 6


def test_splits_for_eight_ranks():
    sys.path.insert(0, ROOT)
    import bench
    assert [bench.strong_shard(32, r, 8) for r in range(8)] == [[4 * r, 4 * r + 4] for r in range(8)]
    assert [bench.by_model_assignment(r, 8) for r in range(8)] == [["resnet50", 4]] * 4 + [["vgg16", 4]] * 4
    assert bench.by_model_assignment(0, 1) is None
    # service mode keeps more shards in rotation the smaller they are
    assert [bench.graphs_in_rotation(n) for n in (32, 16, 8, 4, 1)] == [4, 6, 12, 12, 12]


def test_reference_arm_runs_on_rank_zero_only():
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"], capture_output=True,
                         text=True, timeout=120, env=env, cwd=ROOT)
    assert out.returncode == 0 and out.stdout.strip() == ""
