"""CPU: the reference arm of bench.py (the reference's own CPU code when it is installed under
oracle/_ref, else this repository's restatement of it) prints one JSON line with the keys the
measurement contract asks for, and the GPU arm refuses to run without a device."""

from __future__ import annotations

import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, env=None):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=600, env=dict(os.environ, **(env or {})))


def test_reference_arm_prints_the_contract_line():
    out = _run("--impl", "reference", "--steps", "1", "--warmup", "1")
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "packed_kv_decode_attn_hbm_gbs" and line["unit"] == "GB/s"
    for key in ("value", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["vs_baseline"] is None and line["config"]["workload"]
    cb = line["cpu_baseline"]
    installed = os.path.isfile(os.path.join(ROOT, "oracle", "_ref", "turboquant", "runtime", "packed_qmse_cache.py"))
    assert cb["kind"] == ("reference" if installed else "port")
    assert cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    assert line["steps"] == 1 and line["warmup"] == 1  # K and W are honoured as given
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["value"] > 0


def test_port_and_reference_agree_on_the_output():
    """The two CPU arms compute the same attention (the port is a restatement of the reference):
    checked on a small layer when the reference package is installed.  Runs in a child process:
    the reference shares its import name with this repository's drop-in package."""
    if not os.path.isfile(os.path.join(ROOT, "oracle", "_ref", "turboquant", "runtime", "packed_qmse_cache.py")):
        return
    code = """
import sys, torch
sys.path.insert(0, %r)
import bench
from oracle import tq_oracle as O
ref_cache, ref_attention = bench.load_reference()
k, v, q = O.synth_kvq(1, 8, 2, 300, 128, seed=3, dtype=torch.bfloat16)
layer = ref_cache.PackedMSELayer(bits=4, seed=0, use_qjl_keys=True, quantize_decode=True)
layer.initialize_from_dense(k, v)
theirs = ref_attention.chunked_turboquant_attention(q, layer, n_kv_groups=4)
mine = O.attend_chunked(q, O.pack_layer(k, v, O.QuantParams.build(128, 4, True, seed=0)), 4)
print("SAME" if torch.equal(theirs, mine) else "DIFFERENT")
""" % ROOT
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "SAME" in out.stdout, out.stdout[-500:] + out.stderr[-1500:]


def test_reference_arm_other_ranks_stay_silent():
    out = _run("--impl", "reference", "--gpus", "2", env={"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"})
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_gpu_arm_needs_a_device():
    if torch.cuda.is_available():
        return
    out = _run("--steps", "1", "--warmup", "1")
    assert out.returncode != 0 and "CUDA" in (out.stderr + out.stdout)
