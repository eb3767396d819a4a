"""The N > 1 plumbing of bench.py on CPU: two gloo ranks on the loopback address.

Replicas share nothing on the data path (one runner per GPU, slots never migrate), so what has to
be right is the aggregation: the timed region's duration is the maximum over ranks, the token count
the sum, every rank takes the same amount of work in a different order, and only rank 0 prints.
"""
import json
import os
import socket
import subprocess
import sys
import textwrap

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import json, os, sys
    sys.path.insert(0, os.environ["CARAT_ROOT"])
    import torch
    import bench
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
    torch.distributed.init_process_group("gloo")
    bench.barrier(world)
    maxima, sums = bench.reduce_max_and_sum(world, [10.0 + rank, 5.0 - rank], [100.0 * (rank + 1)])
    contexts, lengths = bench.rank_workload(4, rank)
    bench.barrier(world)
    with open(os.path.join(os.environ["CARAT_OUT"], f"rank{rank}.json"), "w") as out:
        json.dump({"rank": rank, "maxima": maxima, "sums": sums,
                   "lengths": lengths.tolist(), "contexts": contexts}, out)
    torch.distributed.destroy_process_group()
""")


def free_port():
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        return probe.getsockname()[1]


def launch(script_path, out_dir, extra_args=()):
    environment = dict(os.environ, CARAT_ROOT=ROOT, CARAT_OUT=str(out_dir))
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
               "--master-addr", "127.0.0.1", "--master-port", str(free_port()), script_path,
               *extra_args]
    return subprocess.run(command, capture_output=True, text=True, timeout=600, env=environment,
                          cwd=ROOT)


def test_two_ranks_aggregate_max_time_and_sum_tokens(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    done = launch(str(script), tmp_path)
    assert done.returncode == 0, done.stderr[-2000:]
    records = [json.loads((tmp_path / f"rank{rank}.json").read_text()) for rank in (0, 1)]
    assert [record["rank"] for record in records] == [0, 1]
    for record in records:
        assert record["maxima"] == [11.0, 5.0]      # slowest rank's time, per entry
        assert record["sums"] == [300.0]            # tokens of all ranks
    # Each replica serves the same amount of work in an order of its own: the same context
    # lengths on different slots, the same accepted tokens in every step on different slots.
    assert records[0]["lengths"] != records[1]["lengths"]
    assert records[0]["contexts"] != records[1]["contexts"]
    assert sorted(records[0]["contexts"]) == sorted(records[1]["contexts"])
    assert [sorted(row) for row in records[0]["lengths"]] == \
        [sorted(row) for row in records[1]["lengths"]]
    for record in records:
        assert all(1 <= value <= 5 for row in record["lengths"] for value in row)
        assert all(128 <= value <= 6144 for value in record["contexts"])


def test_single_rank_needs_no_process_group():
    sys.path.insert(0, ROOT)
    import bench
    bench.barrier(1)
    assert bench.reduce_max_and_sum(1, [3.0], [4.0]) == ([3.0], [4.0])


def test_accept_lengths_are_seeded_and_bounded():
    sys.path.insert(0, ROOT)
    import bench
    first = bench.accept_lengths(64, seed=7)
    again = bench.accept_lengths(64, seed=7)
    assert torch.equal(first, again)
    assert first.shape == (64, bench.SLOTS)
    assert int(first.min()) >= 1 and int(first.max()) <= bench.DEPTH
    assert 2.0 < float(first.float().mean()) < 3.0   # geometric, mean 2.5, cut at the depth


def test_step_byte_accounting_matches_the_published_figures():
    sys.path.insert(0, ROOT)
    import bench
    import carat_b200
    config = carat_b200.Gemma4Config.gemma4_31b()
    assert bench.step_weight_bytes(config) == 30_696_013_824
    # Full sliding rings (16 KiB per row, 50 layers) plus 8 KiB per context row on 10 global layers.
    positions = [4096] * bench.SLOTS
    per_slot = 50 * 16384 * 1024 + 10 * 8192 * (4096 + bench.DEPTH)
    assert bench.step_kv_bytes(config, positions) == bench.SLOTS * per_slot


def test_clock_sampler_reports_nothing_without_a_gpu_and_decodes_nvml_samples():
    sys.path.insert(0, ROOT)
    import bench
    sampler = bench.ClockSampler(0)
    sampler.start()          # no NVML device and no nvidia-smi here: must not raise
    empty = sampler.stop()
    assert empty["sm_mhz"] is None and empty["reasons"] == []

    # The decoding of NVML samples (clock, reason bit mask), without a device behind it.
    import threading
    decoded = bench.ClockSampler(0)
    decoded.thread = threading.Thread(target=lambda: None)
    decoded.thread.start()
    decoded.stop_flag = threading.Event()
    decoded.maximum = 1965.0
    decoded.samples = [(300.0, 0), (1950.0, 0x4), (1965.0, 0x4), (1965.0, 0)]
    result = decoded.stop()
    assert result["sm_mhz"] == 1965.0 and result["sm_max_mhz"] == 1965.0
    assert result["reasons"] == ["sw_power_cap"] and result["samples"] == 4
