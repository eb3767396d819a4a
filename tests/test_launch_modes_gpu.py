"""The step's results must not depend on how its kernels are launched: with programmatic dependent
launch (the default: the next kernel's prologue overlaps the previous kernel's tail), without it
(CARAT_B200_PDL=0: plain stream order) and with the row kernels as cooperative launches
(CARAT_B200_COOPERATIVE_ROWS=1); nor on whether the largest attention output is found by
the attention kernel or by the quantiser after it (CARAT_B200_ATTENTION_AMAX=0), or on whether
the attention kernel requests its first cache tiles before the previous grid has finished
(CARAT_B200_EARLY_KEYS=0). A kernel that touched another kernel's data before its
griddepcontrol.wait, or a barrier word shared wrongly between launches, would show up as
different tokens between these runs. Full size (31B shapes, 24 slots), each mode in a process
of its own because the switches are read once per process.
"""
import json
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = textwrap.dedent("""
    import json, sys
    sys.path.insert(0, sys.argv[1])
    import torch
    import bench
    config, runner, _ = bench.build_model(seed=0)
    slots = list(range(bench.SLOTS))
    runner.seed_slot_positions(bench.context_lengths(seed=3))
    bench.fill_kv(runner, config, seed=5)
    generator = torch.Generator().manual_seed(4)
    last = torch.randint(3, config.vocabulary_size, (bench.SLOTS,), generator=generator).tolist()
    first = torch.randint(3, config.vocabulary_size, (bench.SLOTS,), generator=generator).tolist()
    record = []
    for step in range(3):
        drafted = runner.draft_four(last, slots, first, bench.DEPTH)
        caps = torch.randint(1, bench.DEPTH + 1, (bench.SLOTS,), generator=generator).tolist()
        result = runner.verify_greedy_proposals(drafted, first, slots, caps, 1)
        record.append([drafted, runner.last_predictions(bench.SLOTS * bench.DEPTH),
                       result.accepted_tokens, result.next_tokens])
        last = [drafted[row][result.accepted_tokens[row] - 1] for row in slots]
        first = result.next_tokens
    following = runner.append_ragged(first, slots)
    print("RESULT " + json.dumps([record, following]))
""")


def run_mode(tmp_path, **switches):
    script = tmp_path / "step.py"
    script.write_text(SCRIPT)
    environment = dict(os.environ)
    for name in ("CARAT_B200_PDL", "CARAT_B200_COOPERATIVE_ROWS", "CARAT_B200_FUSED_GEGLU",
                 "CARAT_B200_ATTENTION_AMAX", "CARAT_B200_EARLY_KEYS"):
        environment.pop(name, None)
    environment.update(switches)
    done = subprocess.run([sys.executable, str(script), ROOT], capture_output=True, text=True,
                          timeout=600, env=environment, cwd=ROOT)
    assert done.returncode == 0, done.stderr[-2000:]
    line = [text for text in done.stdout.splitlines() if text.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


def test_results_do_not_depend_on_the_launch_mode(cuda_device, tmp_path):
    default = run_mode(tmp_path)
    assert run_mode(tmp_path) == default                                   # repeatable at all
    assert run_mode(tmp_path, CARAT_B200_PDL="0") == default
    assert run_mode(tmp_path, CARAT_B200_COOPERATIVE_ROWS="1") == default
    assert run_mode(tmp_path, CARAT_B200_ATTENTION_AMAX="0") == default
    assert run_mode(tmp_path, CARAT_B200_EARLY_KEYS="0") == default
