"""Benchmark of the packed-KV decode-attention hot path.

    python bench.py --gpus N --steps K --warmup W            # this library on N B200s
    python bench.py --impl reference --steps K --warmup W    # the reference algorithm on host cores

Workload (one "step" = one decode step of one attention layer over the whole batch):
Llama-3.1-8B-shaped layer, bf16, 32 query / 8 KV heads, head_dim 128, context 32768,
4-bit Q_prod keys (3-bit Lloyd-Max codes + 1-bit QJL sketch) and 4-bit Q_mse values,
batch 8 per GPU.  K/V are synthetic: iid N(0,1) coordinates with per-token lognormal(0, 0.5)
norms; one N(0,1) query token per sequence.

At N > 1 the KV heads are sharded over the ranks (8/N heads each) and the batch grows to
8*N sequences so every GPU streams the same number of packed bytes (weak scaling); the only
exchange is one NCCL all-gather of the per-head attention outputs per step.

The metric is packed-cache bytes attended per second (134 B per cached token per KV head).
``value`` times the step with everything resident in HBM; ``e2e`` adds, per step, the
host->device copy of the step's inputs (query + the new token's K/V, pinned memory), the
in-place append of that token, and the device->host copy of the attention output (at N > 1
every rank reads back its own heads; the gathered output stays on the devices).

The same line carries a ``model`` block: decode tokens/s of a random-init Llama-3.1-8B (32
layers, bf16) under the library's attention backend at 32768-token context, batch 16, after
a real prompt pass (``prefill_seconds``); at N > 1 the KV heads are sharded, once with the batch
fixed at 16 (``strong``) and once with 16 sequences per GPU (``weak``, caches filled with packed
synthetic K/V).  ``--no-model-block`` leaves it out; ``--gpu-comparator`` adds timings of the
reference's own GPU path (its Triton kernel at batch 1 and its chunked PyTorch path) on the
same GPU when the reference package has been installed into ``oracle/_ref`` (oracle/make_ref.py).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HEAD_DIM = 128
WORKLOAD = dict(name="llama3.1-8b-layer-decode", batch_per_gpu=8, q_heads=32, kv_heads=8, context=32768,
                bits=4, use_qjl=True, dtype="bfloat16")
FALLBACK_HBM_GBS = 6650.0


def bytes_per_unit(bits: int, use_qjl: bool) -> int:
    """Packed bytes read per cached token per KV head in one decode step."""
    key_bits = bits - 1 if use_qjl else bits
    return 16 * key_bits + 2 + (16 + 2 if use_qjl else 0) + 16 * bits + 2


# DRAM bytes (read + write) per unit of the main decode kernel: dram__bytes_read.sum +
# dram__bytes_write.sum of one ncu capture of the CURRENT kernel build on the batch-4 case
# (1 048 576 units of 134 B).  Every packed byte is read once, so traffic grows in proportion to
# the units of a launch.  A constant taken from that capture, not measured by this run: it is
# re-captured whenever the kernel changes, and the line says so (``traffic_kind``).
NCU_TRAFFIC = {"read_bytes": 140.74e6, "write_bytes": 3.79e6, "units": 1048576}
NCU_TRAFFIC_BYTES_PER_UNIT = (NCU_TRAFFIC["read_bytes"] + NCU_TRAFFIC["write_bytes"]) / NCU_TRAFFIC["units"]


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows: list[list[str]] = []
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.rows.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                smax.append(float(r[1]))
            except ValueError:
                continue
            for name, val in zip(names, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------
# CPU arm: the reference's own CPU code when it is installed, else this repository's port of it
# ----------------------------------------------------------------------------

REF_DIR = os.path.join(ROOT, "oracle", "_ref")


def load_reference():
    """The UNMODIFIED reference package from ``oracle/_ref`` (installed by oracle/make_ref.py), or
    None.  It is imported under its own name ``turboquant``; this repository's drop-in package of
    the same name is never imported by the benchmark."""
    if not os.path.isfile(os.path.join(REF_DIR, "turboquant", "runtime", "packed_qmse_cache.py")):
        return None
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    for name in [m for m in sys.modules if m == "turboquant" or m.startswith("turboquant.")]:
        mod_file = getattr(sys.modules[name], "__file__", "") or ""
        if not mod_file.startswith(REF_DIR):
            del sys.modules[name]
    try:
        import turboquant.runtime.attention as ref_attention
        import turboquant.runtime.packed_qmse_cache as ref_cache
    except Exception as exc:  # noqa: BLE001
        print(f"[bench] the reference package in oracle/_ref does not import ({exc!r})", file=sys.stderr)
        return None
    if not (ref_cache.__file__ or "").startswith(REF_DIR):
        return None
    return ref_cache, ref_attention


def cpu_reference_run(steps: int, warmup: int, sample_batch: int = 1):
    """Times chunked decode attention over the packed cache on the host cores (the reference's
    CPU path, src/turboquant/runtime/attention.py:215-304) over a bounded sample of the workload:
    ``sample_batch`` sequence(s) x 8 KV heads x 32768 tokens, all host threads.  Runs the
    reference's own code when it is installed in ``oracle/_ref`` (``kind: "reference"``), else
    this repository's restatement of it (``kind: "port"``)."""
    import torch

    from oracle import tq_oracle as O

    w = WORKLOAD
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    dtype = getattr(torch, w["dtype"])
    groups = w["q_heads"] // w["kv_heads"]
    k, v, q = O.synth_kvq(sample_batch, w["q_heads"], w["kv_heads"], w["context"], HEAD_DIM, seed=0, dtype=dtype)
    ref = load_reference()
    t0 = time.perf_counter()
    if ref is not None:
        ref_cache, ref_attention = ref
        layer = ref_cache.PackedMSELayer(bits=w["bits"], seed=0, use_qjl_keys=w["use_qjl"], quantize_decode=True)
        layer.initialize_from_dense(k, v)
        attend = lambda: ref_attention.chunked_turboquant_attention(q, layer, n_kv_groups=groups)
        kind, what = "reference", "the reference's PackedMSELayer + chunked_turboquant_attention on CPU tensors"
    else:
        p = O.QuantParams.build(HEAD_DIM, w["bits"], w["use_qjl"], seed=0)
        layer = O.pack_layer(k, v, p)
        attend = lambda: O.attend_chunked(q, layer, groups)
        kind, what = "port", "this repository's restatement of the reference's chunked dequantise-then-attend"
    pack_s = time.perf_counter() - t0
    del k, v
    with torch.inference_mode():
        for _ in range(warmup):
            attend()
        t0 = time.perf_counter()
        for _ in range(steps):
            attend()
        dt = (time.perf_counter() - t0) / max(steps, 1)
    nbytes = bytes_per_unit(w["bits"], w["use_qjl"]) * sample_batch * w["kv_heads"] * w["context"]
    return {
        "value": nbytes / dt / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": kind,
        "sample": (f"{sample_batch} of {w['batch_per_gpu']} sequences x {w['kv_heads']} KV heads x {w['context']} "
                   f"tokens, {steps} decode steps after {warmup} warm-up; {what}"),
        "ms_per_step": dt * 1e3, "pack_seconds": pack_s,
        "pack_vectors_per_s": 2 * sample_batch * w["kv_heads"] * w["context"] / pack_s,
    }


def run_self(extra_args: list[str], timeout: float = 900.0):
    """Runs this script in a child process (single GPU, no distributed environment) and returns the
    JSON object of its last output line.  The reference package shares the import name
    ``turboquant`` and the attention-backend name with this library, so everything that imports
    it runs in a process of its own."""
    env = {k: v for k, v in os.environ.items()
           if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT", "LOCAL_WORLD_SIZE",
                        "GROUP_RANK", "ROLE_RANK", "TORCHELASTIC_RUN_ID")}
    try:
        proc = subprocess.run([sys.executable, os.path.abspath(__file__), *extra_args], capture_output=True, text=True,
                              timeout=timeout, env=env)
        lines = [ln for ln in proc.stdout.strip().splitlines() if ln.startswith("{")]
        if proc.returncode != 0 or not lines:
            return {"unavailable": f"child exited {proc.returncode}: {proc.stderr.strip()[-300:]}"}
        return json.loads(lines[-1])
    except Exception as exc:  # noqa: BLE001
        return {"unavailable": repr(exc)[:300]}


def run_reference_arm(args) -> None:
    """``--impl reference``: K steps after W warm-up steps, each step one decode step of one
    sequence of the workload (a bounded sample: the metric is normalised by bytes)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    r = cpu_reference_run(steps, warmup)
    w = WORKLOAD
    line = {
        "impl": "reference", "metric": "packed_kv_decode_attn_hbm_gbs", "value": r["value"], "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["name"], "global_batch": 1, "q_heads": w["q_heads"], "kv_heads": w["kv_heads"],
                   "context": w["context"], "bits": w["bits"], "mode": "Q_prod", "bytes_per_token_head": 134,
                   "sample": "1 of the workload's 8 sequences per step"},
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": r["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------

def synth_on_device(torch, shape, gen, dtype, chunk_tokens=4096):
    """iid N(0,1) coordinates, per-token norm scaled by lognormal(0, 0.5); built in token
    chunks so the fp32 temporaries stay small."""
    b, h, n, d = shape
    out = torch.empty(shape, dtype=dtype, device=gen.device)
    for lo in range(0, n, chunk_tokens):
        hi = min(n, lo + chunk_tokens)
        x = torch.randn(b, h, hi - lo, d, generator=gen, device=gen.device)
        x *= torch.exp(0.5 * torch.randn(b, h, hi - lo, 1, generator=gen, device=gen.device))
        out[:, :, lo:hi] = x.to(dtype)
    return out


def run_gpu_arm(args) -> None:
    import torch
    import torch.distributed as dist

    from tq_local_b200.runtime.codec import Codec
    from tq_local_b200.runtime.packed_store import PackedStore

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path in the product)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    w = dict(WORKLOAD)
    if args.batch_per_gpu:
        w["batch_per_gpu"] = args.batch_per_gpu
    if args.context:
        w["context"] = args.context
    if args.q_heads:
        w["q_heads"] = args.q_heads
    if args.kv_heads:
        w["kv_heads"] = args.kv_heads
    if args.bits:
        w["bits"] = args.bits
    if args.batch_per_gpu or args.context or args.q_heads or args.kv_heads or args.bits:
        w["name"] += " (shape overridden)"
    if w["kv_heads"] % world and world % w["kv_heads"]:
        raise SystemExit(f"{w['kv_heads']} KV heads and {world} ranks: one count must divide the other")
    dtype = getattr(torch, w["dtype"])
    batch = w["batch_per_gpu"] * world
    # fewer KV heads than ranks (e.g. 4 on 8 GPUs): `parts` ranks share each head, each holding a
    # contiguous piece of its tokens; unfinished partials are exchanged instead of outputs
    parts = world // w["kv_heads"] if w["kv_heads"] < world else 1
    hkv = max(1, w["kv_heads"] // world)
    hq = w["q_heads"] // (world // parts)
    n_ctx = w["context"] // parts
    steps, warmup = args.steps, max(args.warmup, 3)
    unit_bytes = bytes_per_unit(w["bits"], w["use_qjl"])

    codec = Codec.get(dev, w["bits"], w["use_qjl"], seed=0)
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    store = PackedStore(codec, batch, hkv, capacity=n_ctx + 2 * (steps + warmup) + 16)
    k = synth_on_device(torch, (batch, hkv, n_ctx, HEAD_DIM), gen, dtype)
    v = synth_on_device(torch, (batch, hkv, n_ctx, HEAD_DIM), gen, dtype)
    store.pack(k, v)  # first call: module load, attribute set-up
    pk0, pk1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    store.length = 0
    torch.cuda.synchronize()
    pk0.record()
    store.pack(k, v)  # the prefill encode of the whole cache, timed warm on the device
    pk1.record()
    torch.cuda.synchronize()
    pack_s = pk0.elapsed_time(pk1) * 1e-3
    del k, v
    q = torch.randn(batch, hq, 1, HEAD_DIM, generator=gen, device=dev).to(dtype)
    out = torch.empty(batch, hq, 1, HEAD_DIM, dtype=dtype, device=dev)
    gathered = torch.empty(world, batch, hq, 1, HEAD_DIM, dtype=dtype, device=dev) if world > 1 else None
    splits = args.splits or store.suggest_splits(n_ctx)
    # N > 1: the per-head outputs are exchanged by the combine kernel itself (stores into the peers'
    # buffers).  If the peer buffers cannot be set up on this box, or a trial step reports a
    # device-side problem on any rank, every rank falls back to an NCCL all-gather.
    peer = None
    if parts > 1:
        from tq_local_b200.runtime.sharding import HeadShard, PeerGather

        peer = PeerGather(HeadShard.from_process_group(), batch, w["q_heads"], dtype, dev, parts=parts)
        args.skip_e2e = True  # (the host-buffer step has no sequence-split form)
    elif world > 1 and args.gather in ("auto", "p2p"):
        from tq_local_b200.runtime.sharding import HeadShard, PeerGather

        ok = torch.ones(1, device=dev)
        try:
            peer = PeerGather(HeadShard.from_process_group(), batch, hq * world, dtype, dev)
        except Exception as exc:  # noqa: BLE001
            print(f"[bench] rank {rank}: peer buffers unavailable ({exc!r})", file=sys.stderr)
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() > 0:
            for _ in range(2):
                store.decode_attn_gather(q, peer, seq_len=n_ctx, splits=splits)
            torch.cuda.synchronize()
            ok.fill_(1.0 if codec.device_status() == 0 else 0.0)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 0:
            if peer is not None:
                peer.close()
            peer = None
            if args.gather == "p2p":
                raise SystemExit("--gather p2p: the peer gather is not usable on this box")

    # One-off, untimed: the fused gather must give, bit for bit, what an NCCL all-gather of the plain
    # decode outputs gives (the only multi-GPU correctness evidence a run on this box can carry).
    gather_check = None
    if world > 1 and peer is not None and parts == 1:
        view = store.decode_attn_gather(q, peer, seq_len=n_ctx, splits=splits)
        store.decode_attn(q, seq_len=n_ctx, splits=splits, out=out)
        dist.all_gather_into_tensor(gathered, out)
        want = gathered.view(world, batch, hq, HEAD_DIM).permute(1, 0, 2, 3).reshape(batch, world * hq, 1, HEAD_DIM)
        torch.cuda.synchronize()
        same = torch.tensor([1.0 if torch.equal(view, want) else 0.0], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        gather_check = "bitexact" if same.item() > 0 else "MISMATCH"

    out_full = torch.empty(batch, w["q_heads"], 1, HEAD_DIM, dtype=dtype, device=dev) if parts > 1 else None

    def step():
        if parts > 1:  # partials of all parts are exchanged, every rank finishes the whole output
            store.decode_attn_parts(q, peer, seq_len=n_ctx, splits=splits, out=out_full)
            return
        if peer is not None:  # the combine kernel writes every rank's gathered buffer itself
            store.decode_attn_gather(q, peer, seq_len=n_ctx, splits=splits)
            return
        store.decode_attn(q, seq_len=n_ctx, splits=splits, out=out)
        if world > 1:
            dist.all_gather_into_tensor(gathered, out)

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing (measurement hooks off)
    for _ in range(warmup):
        step()
    fence()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fence()
    ev0.record()
    for _ in range(steps):
        step()
    ev1.record()
    fence()
    ms = ev0.elapsed_time(ev1) / steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())

    # ---- same steps again, straight after the timed ones (same clocks), with the library's hooks
    # on: CUDA events around the main kernel (on its launch stream) give the roofline numerator;
    # every launch is counted
    codec.profile(True)
    fence()
    for _ in range(steps):
        step()
    fence()
    main_ms, main_n, all_launches = codec.profile_read()
    codec.profile(False)

    # The timed region lasts a few milliseconds, too short for more than one clock sample: keep the
    # identical steps running (untimed) for about half a second so that the clock / throttle record
    # describes this load.  (Same count on every rank: the steps synchronise the ranks.)
    for _ in range(min(20000, max(steps, int(0.5 / max(ms * 1e-3, 1e-6))))):
        step()
    fence()

    # ---- end to end: host buffers in, host buffer out, one new token appended per step
    pin = dict(dtype=dtype, pin_memory=True)
    h_q = torch.randn(batch, hq, 1, HEAD_DIM).to(dtype).pin_memory()
    h_k = (torch.randn(batch, hkv, 1, HEAD_DIM)).to(dtype).pin_memory()
    h_v = (torch.randn(batch, hkv, 1, HEAD_DIM)).to(dtype).pin_memory()
    h_out = torch.empty(batch, hq, 1, HEAD_DIM, **pin)  # N > 1: this rank's heads (the gathered output stays on the devices)
    d_q, d_k, d_v = torch.empty_like(q), torch.empty(batch, hkv, 1, HEAD_DIM, dtype=dtype, device=dev), \
        torch.empty(batch, hkv, 1, HEAD_DIM, dtype=dtype, device=dev)
    h2d = h_q.numel() * h_q.element_size() + h_k.numel() * h_k.element_size() + h_v.numel() * h_v.element_size()
    d2h = out.numel() * out.element_size()

    h_out1 = torch.empty(batch, hq, 1, HEAD_DIM, **pin)
    host_step = store.bind_host_step(h_q, h_k, h_v, h_out1) if world == 1 else None

    def e2e_step():
        if world == 1:
            # the library's host-buffer entry point: H2D of q / k / v, append, attend, D2H of the output
            host_step()
        elif peer is not None:
            # shard: host buffers in, gathered output of all ranks straight into the host buffer
            store.decode_step_host_gather(h_q, h_k, h_v, h_out, peer)
        else:
            d_q.copy_(h_q, non_blocking=True)
            d_k.copy_(h_k, non_blocking=True)
            d_v.copy_(h_v, non_blocking=True)
            store.pack(d_k, d_v)
            store.decode_attn(d_q, splits=splits, out=out)
            dist.all_gather_into_tensor(gathered, out)
            h_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the host needs the result before the next token

    e2e_steps = 0 if args.skip_e2e else steps
    for _ in range(0 if args.skip_e2e else warmup):
        e2e_step()
    fence()
    ev0.record()
    for _ in range(e2e_steps):
        e2e_step()
    ev1.record()
    fence()
    e2e_ms = ev0.elapsed_time(ev1) / max(e2e_steps, 1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    clocks = sampler.stop() if rank == 0 else None

    # ---- context figure: the same decode step over a DENSE bf16 cache with torch's SDPA (what the
    # reference calls its baseline), N = 1 only; the dense cache is 3.8x the packed bytes
    dense = None
    if world == 1 and not args.skip_e2e:
        try:
            import torch.nn.functional as F

            dk = torch.randn(batch, hkv, n_ctx, HEAD_DIM, device=dev, dtype=dtype)
            dv = torch.randn(batch, hkv, n_ctx, HEAD_DIM, device=dev, dtype=dtype)
            for _ in range(3):
                F.scaled_dot_product_attention(q, dk, dv, enable_gqa=True)
            torch.cuda.synchronize()
            ev0.record()
            for _ in range(10):
                F.scaled_dot_product_attention(q, dk, dv, enable_gqa=True)
            ev1.record()
            torch.cuda.synchronize()
            dense_ms = ev0.elapsed_time(ev1) / 10
            dense = {"ms_per_step": dense_ms, "dense_bytes": 2 * dk.numel() * dk.element_size(),
                     "dense_gbs": 2 * dk.numel() * dk.element_size() / (dense_ms * 1e-3) / 1e9,
                     "what": "torch scaled_dot_product_attention over the same keys/values kept dense in bf16"}
            del dk, dv
        except Exception as exc:  # noqa: BLE001
            dense = {"unavailable": repr(exc)}

    if rank == 0:
        units_total = batch * hkv * n_ctx * world  # every rank attends batch x hkv rows
        total_bytes = unit_bytes * units_total
        per_launch_bytes = unit_bytes * batch * hkv * n_ctx
        peak, peak_src = measured_peak()
        achieved = per_launch_bytes / (main_ms / max(main_n, 1) * 1e-3) / 1e9 if main_n else None
        line = {
            "metric": "packed_kv_decode_attn_hbm_gbs", "value": total_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": w["name"], "global_batch": batch, "q_heads": w["q_heads"], "kv_heads": w["kv_heads"],
                "context": w["context"], "bits": w["bits"], "mode": "Q_prod", "bytes_per_token_head": unit_bytes,
                "parallelism": (f"kv-head-shard{world // parts} x sequence-split{parts}, partials exchanged by peer stores"
                                if parts > 1 else
                                f"kv-head-shard{world}, outputs gathered by "
                                + ("peer stores from the combine kernel" if peer is not None else "NCCL all-gather"))
                if world > 1 else "single",
                "splits": splits, "l2": f"inputs larger than L2 ({unit_bytes * batch * hkv * n_ctx / 1e6:.0f} MB of packed cache per GPU per step vs 126 MB)",
            },
            "decode_tok_per_s_layer": batch / (ms * 1e-3),
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": (achieved / peak) if achieved else None, "peak_source": f"of {peak_src}",
                "kernel": "tq_decode main kernel (streams the packed cache)",
                "kernel_ms": main_ms / max(main_n, 1),
                "traffic": NCU_TRAFFIC_BYTES_PER_UNIT * batch * hkv * n_ctx if w["bits"] == 4 and hq // hkv <= 4 else None,
                "traffic_kind": ("constant: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this "
                                 "kernel build on the batch-4 case, scaled by the units of a launch; not measured by "
                                 "this run"),
            },
            "e2e": None if args.skip_e2e else {
                "value": total_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(all_launches),
            "device_status": codec.device_status(),
            "clocks": dict(clocks or {}, window="the timed steps and ~0.5 s of the same steps kept running after them, "
                                                "the hooked steps and the end-to-end steps"),
            "pack": {"seconds": pack_s, "vectors_per_s": 2 * batch * hkv * n_ctx / pack_s},
            "dense_sdpa": dense,
        }
        if gather_check is not None:
            line["gather_check"] = gather_check
        if world == 1 and not args.no_cpu_baseline:
            cb = run_self(["--impl", "reference", "--steps", "3", "--warmup", "1"]).get("cpu_baseline")
            line["cpu_baseline"] = cb if cb else {"unavailable": "the CPU arm did not run"}
    else:
        line = None
    if peer is not None:
        peer.close()
    # free the layer workload before the whole-model block and the comparator
    del store, q, out, gathered
    torch.cuda.empty_cache()
    if args.gpu_comparator and world == 1 and rank == 0:
        line["gpu_comparator"] = run_self(["--gpu-comparator-only"])
    if not args.no_model_block:
        try:
            block = model_block(args, torch, dist, world, rank, local_rank, dev)
        except Exception as exc:  # noqa: BLE001  (the headline line must still be printed)
            if world > 1:
                raise
            block = {"unavailable": repr(exc)[:300]}
        if rank == 0:
            line["model"] = block
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ----------------------------------------------------------------------------
# Whole-model decode: random-init Llama-3.1-8B over 32k-token packed caches
# ----------------------------------------------------------------------------

MODEL_WORKLOAD = dict(name="llama3.1-8b-random-init-decode", batch=16, context=32768, layers=32, hidden=4096,
                      intermediate=14336, q_heads=32, kv_heads=8, vocab=128256, bits=4, use_qjl=True)


def build_model(torch, w, dev):
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=w["vocab"], hidden_size=w["hidden"], intermediate_size=w["intermediate"],
                      num_hidden_layers=w["layers"], num_attention_heads=w["q_heads"],
                      num_key_value_heads=w["kv_heads"], head_dim=HEAD_DIM, max_position_embeddings=131072,
                      tie_word_embeddings=False)
    torch.manual_seed(0)
    old_dtype = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            return LlamaForCausalLM(cfg).eval()
    finally:
        torch.set_default_dtype(old_dtype)


def model_decode_run(torch, dist, model, w, shard, world, rank, local_rank, dev, steps, warmup, batch, real_prefill):
    """Decode tokens/s of the whole model at ``batch`` sequences x ``w['context']`` tokens: the packed
    caches come from a real prompt pass over random token ids (``real_prefill``: a streaming prefill in
    row blocks, timed as ``prefill_seconds``) or are filled with packed synthetic K/V; then greedy
    decoding through the library's attention backend, the model step replayed from a CUDA graph
    (KV-head shards exchange their outputs through the fused peer gather inside the recorded step).
    Timed with CUDA events over ``steps`` steps after ``warmup``, maximum over the ranks."""
    from transformers.cache_utils import Cache

    from tq_local_b200.adapters.transformers import disable_turboquant_attention, enable_turboquant_attention
    from tq_local_b200.runtime import generation
    from tq_local_b200.runtime.packed_qmse_cache import PackedMSELayer, build_streaming_prefill_cache

    gen = torch.Generator(device=dev).manual_seed(99)
    B, N = batch, w["context"]

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    prefill_s = None
    with torch.inference_mode():
        if real_prefill:
            ids = torch.randint(0, w["vocab"], (B, N), device=dev, generator=gen)
            cache = build_streaming_prefill_cache(w["layers"], w["bits"], head_dim=HEAD_DIM, use_qjl_keys=w["use_qjl"],
                                                  quantize_decode=True, norm_guard=True,
                                                  reserve_tokens=steps + warmup + 8, shard=shard)
            rows = max(1, generation.PREFILL_BLOCK_TOKENS // N)
            fence()
            t0 = time.perf_counter()
            last = generation._prefill_in_row_blocks(model, {"input_ids": ids}, cache,
                                                     generation._auto_norm_threshold(w["bits"], HEAD_DIM), rows)
            first = torch.argmax(last, dim=-1, keepdim=True)
            fence()
            prefill_s = time.perf_counter() - t0
            if world > 1:
                t = torch.tensor([prefill_s], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                prefill_s = float(t.item())
            layers = cache.layers
            del ids, last
        else:
            layers = []
            for _ in range(w["layers"]):
                k = synth_on_device(torch, (B, w["kv_heads"], N, HEAD_DIM), gen, torch.bfloat16)
                v = synth_on_device(torch, (B, w["kv_heads"], N, HEAD_DIM), gen, torch.bfloat16)
                layer = PackedMSELayer(bits=w["bits"], use_qjl_keys=w["use_qjl"], quantize_decode=True,
                                       reserve_tokens=steps + warmup + 8, shard=shard)
                layer.initialize_from_dense(k, v)
                layers.append(layer)
                del k, v
            cache = Cache(layers=layers)
            first = torch.randint(0, w["vocab"], (B, 1), device=dev, generator=gen)
        dense_layers = sum(1 for layer in layers if layer._force_dense)
        for layer in layers:
            layer.bind_attention_mask(None, lock=True)  # no padding: the layers need not look at per-call masks
        old_impl = enable_turboquant_attention(model, cache)
        sampler = ClockSampler(local_rank)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        try:
            q_heads = w["q_heads"]
            if all(layer.supports_static_decode(q_heads) for layer in layers):
                with generation.RecordedDecoder(model, cache, first, warmup + steps) as dec:
                    for _ in range(warmup):
                        dec.step()
                    fence()
                    if rank == 0:
                        sampler.start()
                    ev0.record()
                    for _ in range(steps):
                        dec.step()
                    ev1.record()
                    fence()
                    recorded = bool(dec.graph)
                    tokens = dec.tokens.clone()
            else:
                recorded, produced, tok = False, [], first

                def eager_step(tok):
                    out = model(input_ids=tok, past_key_values=cache, use_cache=True)
                    return torch.argmax(out.logits[:, -1, :], dim=-1, keepdim=True)

                for _ in range(warmup):
                    tok = eager_step(tok)
                fence()
                if rank == 0:
                    sampler.start()
                ev0.record()
                for _ in range(steps):
                    tok = eager_step(tok)
                    produced.append(tok)
                ev1.record()
                fence()
                tokens = torch.cat(produced, dim=-1)
        finally:
            disable_turboquant_attention(model, cache, old_impl)
    ms = ev0.elapsed_time(ev1) / steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    clocks = sampler.stop() if rank == 0 else None
    unit = bytes_per_unit(w["bits"], w["use_qjl"])
    packed_bytes = unit * B * w["kv_heads"] * N * (w["layers"] - dense_layers)
    weight_bytes = sum(p.numel() * p.element_size() for p in model.parameters())
    status = max((layer.codec.device_status() for layer in layers if layer.codec is not None), default=0)
    result = {
        "tok_per_s": B * 1e3 / ms, "ms_per_step": ms, "global_batch": B, "steps": steps, "warmup": warmup,
        "prefill_seconds": prefill_s,
        "prefill": ("real prompt pass over random token ids, streamed into the packed cache in row blocks"
                    if real_prefill else "caches filled with packed synthetic K/V (no prompt pass)"),
        "decode_step": "CUDA graph replay" if recorded else "eager",
        "packed_kv_bytes_per_step": packed_bytes, "weight_bytes": weight_bytes,
        "hbm_gbs_lower_bound": (packed_bytes / world + weight_bytes) / (ms * 1e-3) / 1e9,
        "tokens_checksum": int(tokens.sum().item()), "device_status": status, "clocks": clocks,
    }
    del cache, layers
    torch.cuda.empty_cache()
    return result


def model_block(args, torch, dist, world, rank, local_rank, dev):
    """The ``model`` block of the benchmark line (see the module docstring)."""
    from tq_local_b200.runtime.sharding import HeadShard

    w = dict(MODEL_WORKLOAD)
    if args.context:
        w["context"] = args.context
    if args.layers:
        w["layers"] = args.layers
    steps, warmup = max(4, min(args.steps, 32)), 3
    shard = HeadShard.from_process_group() if world > 1 else HeadShard()
    model = build_model(torch, w, dev)
    block = {"workload": w["name"], "context": w["context"], "layers": w["layers"], "metric": "decode_tok_per_s_32k_ctx",
             "unit": "tok/s", "parallelism": f"kv-head-shard{world}, weights replicated" if world > 1 else "single"}
    block["strong"] = model_decode_run(torch, dist, model, w, shard, world, rank, local_rank, dev, steps, warmup,
                                       w["batch"], real_prefill=not args.synthetic_prefill)
    block["strong"]["scaling"] = "strong (batch 16 in total)"
    if world > 1:
        block["weak"] = model_decode_run(torch, dist, model, w, shard, world, rank, local_rank, dev, steps, warmup,
                                         w["batch"] * world, real_prefill=False)
        block["weak"]["scaling"] = "weak (16 sequences per GPU)"
    else:
        block["weak"] = dict(block["strong"], scaling="weak (16 sequences per GPU; the same run at one GPU)")
    del model
    torch.cuda.empty_cache()
    return block


def run_model_arm(args) -> None:
    """``--workload model``: the whole-model figure alone, as a line of its own."""
    import torch
    import torch.distributed as dist

    from tq_local_b200.runtime.sharding import HeadShard

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    w = dict(MODEL_WORKLOAD)
    if args.batch_per_gpu:
        w["batch"] = args.batch_per_gpu
    if args.model_scaling == "weak":
        w["batch"] *= world  # every GPU then streams the same packed bytes as one GPU does at N = 1
    if args.context:
        w["context"] = args.context
    if args.layers:
        w["layers"] = args.layers
    steps, warmup = args.steps, max(args.warmup, 3)
    shard = HeadShard.from_process_group() if world > 1 else HeadShard()
    model = build_model(torch, w, dev)
    r = model_decode_run(torch, dist, model, w, shard, world, rank, local_rank, dev, steps, warmup, w["batch"],
                         real_prefill=not args.synthetic_prefill and args.model_scaling == "strong")
    if rank == 0:
        line = {
            "metric": "decode_tok_per_s_32k_ctx", "value": r["tok_per_s"], "unit": "tok/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
            "scaling": args.model_scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["name"], "global_batch": w["batch"], "context": w["context"], "layers": w["layers"],
                       "q_heads": w["q_heads"], "kv_heads": w["kv_heads"], "bits": w["bits"], "mode": "Q_prod",
                       "parallelism": f"kv-head-shard{world}, weights replicated" if world > 1 else "single",
                       "decode_step": r["decode_step"], "prefill": r["prefill"]},
        }
        line.update({k: r[k] for k in ("prefill_seconds", "packed_kv_bytes_per_step", "weight_bytes",
                                       "hbm_gbs_lower_bound", "tokens_checksum", "device_status", "clocks")})
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ----------------------------------------------------------------------------
# The reference's own GPU path on the same GPU (comparator only; never on the product's path)
# ----------------------------------------------------------------------------

def gpu_comparator(torch, dev, steps: int = 10):
    """Times the reference's fused Triton decode attention (batch 1: the only shape it serves,
    src/turboquant/runtime/triton_kernels.py:238-368) and its chunked PyTorch path on the GPU
    (batch 8, src/turboquant/runtime/attention.py:215-304) at the workload's shape, with the
    reference package from ``oracle/_ref``.  CUDA events, 3 warm-up calls."""
    ref = load_reference()
    if ref is None:
        return {"unavailable": "the reference package is not installed in oracle/_ref (python oracle/make_ref.py)"}
    ref_cache, ref_attention = ref
    import turboquant.runtime.triton_kernels as ref_tk

    w = WORKLOAD
    dtype = getattr(torch, w["dtype"])
    groups = w["q_heads"] // w["kv_heads"]
    gen = torch.Generator(device=dev).manual_seed(4321)
    unit = bytes_per_unit(w["bits"], w["use_qjl"])
    out = {}
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for name, batch in (("triton_fused_batch1", 1), ("chunked_pytorch_batch8", w["batch_per_gpu"])):
        try:
            with torch.inference_mode():
                layer = ref_cache.PackedMSELayer(bits=w["bits"], seed=0, use_qjl_keys=w["use_qjl"], quantize_decode=True)
                k = synth_on_device(torch, (batch, w["kv_heads"], w["context"], HEAD_DIM), gen, dtype)
                v = synth_on_device(torch, (batch, w["kv_heads"], w["context"], HEAD_DIM), gen, dtype)
                layer.initialize_from_dense(k, v)
                del k, v
                q = torch.randn(batch, w["q_heads"], 1, HEAD_DIM, generator=gen, device=dev).to(dtype)
                if name.startswith("triton"):
                    call = lambda: ref_tk.fused_attention(q, layer, groups)
                    if call() is None:
                        out[name] = {"unavailable": "fused_attention returned None (Triton path not taken)"}
                        continue
                else:
                    call = lambda: ref_attention.chunked_turboquant_attention(q, layer, n_kv_groups=groups)
                for _ in range(3):
                    call()
                torch.cuda.synchronize()
                ev0.record()
                for _ in range(steps):
                    call()
                ev1.record()
                torch.cuda.synchronize()
                ms = ev0.elapsed_time(ev1) / steps
                nbytes = unit * batch * w["kv_heads"] * w["context"]
                out[name] = {"ms_per_step": ms, "packed_gbs": nbytes / (ms * 1e-3) / 1e9, "batch": batch,
                             "what": ("the reference's fused_attention (Triton tile kernel + host-side reduce)"
                                      if name.startswith("triton") else
                                      "the reference's chunked_turboquant_attention on CUDA tensors (what it runs "
                                      "for batch > 1)")}
                del layer
                torch.cuda.empty_cache()
        except Exception as exc:  # noqa: BLE001
            out[name] = {"unavailable": repr(exc)[:300]}
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch-per-gpu", type=int, default=None,
                    help="override the workload's batch (profiling captures use a smaller one)")
    ap.add_argument("--context", type=int, default=None, help="override the context length (profiling captures)")
    ap.add_argument("--q-heads", type=int, default=None, help="override the query-head count (profiling captures)")
    ap.add_argument("--kv-heads", type=int, default=None, help="override the KV-head count (profiling captures)")
    ap.add_argument("--bits", type=int, default=None, choices=[2, 3, 4], help="override the bit width (profiling captures)")
    ap.add_argument("--splits", type=int, default=None, help="override the library's split choice")
    ap.add_argument("--skip-e2e", action="store_true", help="device-resident timing only (profiling captures)")
    ap.add_argument("--workload", default="layer", choices=["layer", "model"],
                    help="layer: one attention layer's decode step (the headline metric); model: whole-model "
                         "decode tokens/s of a random-init Llama-3.1-8B over 32k-token packed caches")
    ap.add_argument("--gather", default="auto", choices=["auto", "nccl", "p2p"],
                    help="N > 1: how the per-head outputs are exchanged: p2p = stores into the peers' buffers fused "
                         "into the combine kernel, nccl = NCCL all-gather, auto = p2p with a fall-back to nccl")
    ap.add_argument("--model-scaling", default="strong", choices=["strong", "weak"],
                    help="model workload at N > 1: strong = batch 16 in total, weak = 16 sequences per GPU")
    ap.add_argument("--layers", type=int, default=None, help="model workload: override the layer count (smoke runs)")
    ap.add_argument("--no-model-block", action="store_true",
                    help="layer workload: leave the whole-model block out of the line (profiling captures)")
    ap.add_argument("--synthetic-prefill", action="store_true",
                    help="model workload: fill the caches with packed synthetic K/V instead of running the prompt pass")
    ap.add_argument("--gpu-comparator", action="store_true",
                    help="N = 1: also time the reference's own GPU path (needs oracle/_ref, see oracle/make_ref.py)")
    ap.add_argument("--gpu-comparator-only", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.gpu_comparator_only:
        import torch

        print(json.dumps(gpu_comparator(torch, torch.device("cuda", 0))))
    elif args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "model":
        run_model_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
