"""bench.py without a GPU: the command line the driver uses parses, the GPU arm
refuses to run (there is no CPU path) with one JSON line on stdout and nothing
else there, and the ranks of the reference arm other than 0 exit without
work."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(args, env=None):
    e = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    e.update(env or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=300, env=e)


def test_gpu_arm_refuses_without_a_device():
    res = run(["--gpus", "1", "--steps", "20", "--warmup", "5"])
    assert res.returncode == 1
    lines = [l for l in res.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "no CPU path" in json.loads(lines[0])["error"]


def test_reference_arm_runs_on_rank_zero_only():
    res = run(["--impl", "reference", "--gpus", "2", "--steps", "2", "--warmup", "1"], env={"RANK": "1", "WORLD_SIZE": "2"})
    assert res.returncode == 0 and res.stdout.strip() == ""


def test_defaults_are_the_sharded_configuration():
    sys.path.insert(0, ROOT)
    import bench

    old = sys.argv
    sys.argv = ["bench.py"]
    try:
        a = bench.parse_args()
    finally:
        sys.argv = old
    assert (a.gpus, a.workload, a.impl, a.redistribution) == (1, 3, "b200", "p2p")
    assert a.steps * a.batches_per_step * 64 >= 128 * 100   # a default run times well over a hundred steps' worth of calls
    assert set(bench.TRAFFIC) == {0, 1, 2, 3}
    for v in bench.TRAFFIC.values():
        assert os.path.exists(os.path.join(ROOT, v["source"]))


def test_gpus_n_without_a_launcher_starts_n_ranks():
    """``python bench.py --gpus 2`` re-executes itself under torch.distributed.run;
    without a device each of the two ranks refuses with its own line."""
    env = {k: None for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT")}
    e = {k: v for k, v in dict(os.environ, CUDA_VISIBLE_DEVICES="").items() if k not in env}
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=300, env=e)
    assert res.returncode != 0
    lines = [l for l in res.stdout.splitlines() if l.strip().startswith("{")]
    assert len(lines) == 2 and all("no CPU path" in json.loads(l)["error"] for l in lines)
