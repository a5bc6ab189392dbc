"""Host logic of the multi-GPU benchmark, on CPU: two ``gloo`` ranks stand in for two GPUs.

The data path has no collective (independent replicas); what N > 1 adds is the max-over-ranks
of the timing scalars, per-rank seeds, rank 0 printing alone, and the reference arm running on
rank 0 only.
"""

import json
import os
import subprocess
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def _rank_main(rank: int, world: int, port: int, out_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world))
    import bench

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # rank 1 is the slow replica for the device time, rank 0 for the end-to-end time
        device_ms, e2e_ms = bench.max_over_ranks([10.0 + 5.0 * rank, 40.0 - 7.0 * rank], "cpu", True)
        # every replica draws its own weights and token ids
        g = torch.Generator().manual_seed(7 + rank)
        ids = torch.randint(0, 1000, (4,), generator=g)
        gathered = [torch.zeros_like(ids) for _ in range(world)]
        dist.all_gather(gathered, ids)
        result = {"device_ms": device_ms, "e2e_ms": e2e_ms,
                  "ids_differ": not torch.equal(gathered[0], gathered[1]),
                  "tokens_per_s": bench.whole_job_rate(8, world, device_ms * 1e-3)}
        Path(out_dir, f"rank{rank}.json").write_text(json.dumps(result))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_ranks_agree_on_the_slowest_replica(tmp_path):
    port = 29500 + os.getpid() % 2000
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    results = [json.loads((tmp_path / f"rank{r}.json").read_text()) for r in range(2)]
    for r in results:
        assert r["device_ms"] == 15.0 and r["e2e_ms"] == 40.0     # max over ranks, on every rank
        assert r["ids_differ"]
        assert r["tokens_per_s"] == 8 * 2 / 15e-3                 # whole-job rate, weak scaling


def _run_reference(rank: int) -> subprocess.CompletedProcess:
    env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank),
               MASTER_ADDR="127.0.0.1", MASTER_PORT="29999")
    return subprocess.run(
        [sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2",
         "--workload", "smollm-135m-b1-k32", "--steps", "1", "--warmup", "1"],
        env=env, capture_output=True, text=True, timeout=600)


def test_reference_arm_runs_on_rank_zero_only():
    silent = _run_reference(1)
    assert silent.returncode == 0 and silent.stdout.strip() == ""
    spoken = _run_reference(0)
    assert spoken.returncode == 0, spoken.stderr[-2000:]
    line = json.loads(spoken.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["n_gpus"] == 2
    assert line["metric"] == "decode_us_per_token" and line["unit"] == "us/token"
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["value"] > 0


def test_both_arms_describe_the_workload_identically():
    """The reference arm and the GPU arm print the same ``config`` for the same command line."""
    import bench

    for name in ("qwen2-0.5b-b8-k4096", "smollm-135m-b1-k32"):
        config = bench.decode_config(name, 2, "prefill")
        assert set(config) == {"workload", "model", "batch_per_gpu", "cached_keys", "replicas",
                               "parallelism", "weights", "cache_fill", "l2"}
        assert config["replicas"] == 2 and config["workload"] == name
    spoken = _run_reference(0)
    line = json.loads(spoken.stdout.strip().splitlines()[-1])
    assert line["config"] == bench.decode_config("smollm-135m-b1-k32", 2, "prefill")
    assert line["steps"] == 1 and line["warmup"] == 3 and line["steps_timed"] >= 1
    prefill = bench.prefill_config("gemma-2b-prefill-t128", 1)
    assert prefill["prompt_tokens"] == 128 and prefill["model"] == "gemma-2b"
