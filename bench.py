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
in-place append of that token, and the device->host copy of the attention output.
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


# DRAM bytes (read + write) per unit of the main decode kernel, from the ncu capture of the
# batch-4 case summarised in profiles/decode_mma4_b4_ctx32768.md: 140.74 MB read +
# 3.6 MB written for 1 048 576 units of 134 B.  Every packed byte is read once, so traffic
# grows in proportion to the units of a launch.
NCU_TRAFFIC_BYTES_PER_UNIT = (140.74e6 + 3.6e6) / 1048576


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
# CPU arm: the reference algorithm (oracle port) on the host cores
# ----------------------------------------------------------------------------

def cpu_reference_run(steps: int, warmup: int, sample_batch: int = 1):
    """Times the oracle's chunked decode attention (the reference's CPU path,
    src/turboquant/runtime/attention.py:215-304) over a bounded sample of the workload:
    ``sample_batch`` sequence(s) x 8 KV heads x 32768 tokens, all host threads."""
    import torch

    from oracle import tq_oracle as O

    w = WORKLOAD
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    dtype = getattr(torch, w["dtype"])
    groups = w["q_heads"] // w["kv_heads"]
    k, v, q = O.synth_kvq(sample_batch, w["q_heads"], w["kv_heads"], w["context"], HEAD_DIM, seed=0, dtype=dtype)
    p = O.QuantParams.build(HEAD_DIM, w["bits"], w["use_qjl"], seed=0)
    t0 = time.perf_counter()
    layer = O.pack_layer(k, v, p)
    pack_s = time.perf_counter() - t0
    del k, v
    for _ in range(warmup):
        O.attend_chunked(q, layer, groups)
    t0 = time.perf_counter()
    for _ in range(steps):
        O.attend_chunked(q, layer, groups)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    nbytes = bytes_per_unit(w["bits"], w["use_qjl"]) * sample_batch * w["kv_heads"] * w["context"]
    return {
        "value": nbytes / dt / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
        "sample": (f"{sample_batch} of {w['batch_per_gpu']} sequences x {w['kv_heads']} KV heads x {w['context']} "
                   f"tokens, {steps} decode steps after {warmup} warm-up (chunked dequantise-then-attend)"),
        "ms_per_step": dt * 1e3, "pack_seconds": pack_s,
        "pack_vectors_per_s": 2 * sample_batch * w["kv_heads"] * w["context"] / pack_s,
    }


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, min(args.steps, 8)), max(1, min(args.warmup, 2))
    r = cpu_reference_run(steps, warmup)
    w = WORKLOAD
    line = {
        "impl": "reference", "metric": "packed_kv_decode_attn_hbm_gbs", "value": r["value"], "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["name"], "batch": 1, "q_heads": w["q_heads"], "kv_heads": w["kv_heads"],
                   "context": w["context"], "bits": w["bits"], "mode": "Q_prod", "bytes_per_token_head": 134},
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
    if w["kv_heads"] % world:
        raise SystemExit(f"{w['kv_heads']} KV heads do not shard over {world} ranks")
    dtype = getattr(torch, w["dtype"])
    batch = w["batch_per_gpu"] * world
    hkv = w["kv_heads"] // world
    hq = w["q_heads"] // world
    n_ctx = w["context"]
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
    if world > 1 and args.gather in ("auto", "p2p"):
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

    def step():
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

    # The timed region lasts a few milliseconds, too short for more than one clock sample: keep the
    # identical steps running (untimed) for about half a second so that the clock / throttle record
    # describes this load.  (Same count on every rank: the steps synchronise the ranks.)
    for _ in range(min(20000, max(steps, int(0.5 / max(ms * 1e-3, 1e-6))))):
        step()
    fence()

    # ---- same steps again with the library's hooks on: CUDA events around the main kernel
    # (on its launch stream) give the roofline numerator; every launch is counted
    codec.profile(True)
    fence()
    for _ in range(steps):
        step()
    fence()
    main_ms, main_n, all_launches = codec.profile_read()
    codec.profile(False)

    # ---- end to end: host buffers in, host buffer out, one new token appended per step
    pin = dict(dtype=dtype, pin_memory=True)
    h_q = torch.randn(batch, hq, 1, HEAD_DIM).to(dtype).pin_memory()
    h_k = (torch.randn(batch, hkv, 1, HEAD_DIM)).to(dtype).pin_memory()
    h_v = (torch.randn(batch, hkv, 1, HEAD_DIM)).to(dtype).pin_memory()
    h_out = torch.empty(batch, hq * world, 1, HEAD_DIM, **pin)
    d_q, d_k, d_v = torch.empty_like(q), torch.empty(batch, hkv, 1, HEAD_DIM, dtype=dtype, device=dev), \
        torch.empty(batch, hkv, 1, HEAD_DIM, dtype=dtype, device=dev)
    h2d = h_q.numel() * h_q.element_size() + h_k.numel() * h_k.element_size() + h_v.numel() * h_v.element_size()
    d2h = (gathered if world > 1 else out).numel() * out.element_size()

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
            h_out.view(batch, world, hq, HEAD_DIM).copy_(
                gathered.view(world, batch, hq, HEAD_DIM).transpose(0, 1), non_blocking=True)
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
                "context": n_ctx, "bits": w["bits"], "mode": "Q_prod", "bytes_per_token_head": unit_bytes,
                "parallelism": (f"kv-head-shard{world}, outputs gathered by "
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
                "traffic": NCU_TRAFFIC_BYTES_PER_UNIT * batch * hkv * n_ctx if w["bits"] == 4 else None,
                "traffic_source": "ncu dram read+write of the batch-4 capture in profiles/, scaled by units",
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
        if world == 1 and not args.no_cpu_baseline:
            cb = cpu_reference_run(steps=3, warmup=1)
            line["cpu_baseline"] = {k_: cb[k_] for k_ in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    if peer is not None:
        peer.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ----------------------------------------------------------------------------
# Whole-model decode: random-init Llama-3.1-8B over a packed 32k-token cache
# ----------------------------------------------------------------------------

MODEL_WORKLOAD = dict(name="llama3.1-8b-random-init-decode", batch=16, context=32768, layers=32, hidden=4096,
                      intermediate=14336, q_heads=32, kv_heads=8, vocab=128256, bits=4, use_qjl=True)


def run_model_arm(args) -> None:
    """Decode tokens/s of a whole model step: random-init Llama-3.1-8B (bf16), batch 16, every
    layer's cache holding 32768 packed tokens per sequence (4-bit Q_prod), greedy decoding through
    the library's attention backend with the model step replayed from a CUDA graph.  The caches
    are filled with packed synthetic K/V (the prompt pass is not part of a decode-rate figure).
    At N > 1 the weights are replicated and the KV heads are sharded (outputs exchanged by the
    fused peer gather inside the recorded step); the batch stays 16 (``--model-scaling strong``) or
    grows with N (``weak``)."""
    import torch
    import torch.distributed as dist
    from transformers import LlamaConfig, LlamaForCausalLM
    from transformers.cache_utils import Cache

    from tq_local_b200.adapters.transformers import disable_turboquant_attention, enable_turboquant_attention
    from tq_local_b200.runtime.generation import RecordedDecoder
    from tq_local_b200.runtime.packed_qmse_cache import PackedMSELayer
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
    cfg = LlamaConfig(vocab_size=w["vocab"], hidden_size=w["hidden"], intermediate_size=w["intermediate"],
                      num_hidden_layers=w["layers"], num_attention_heads=w["q_heads"],
                      num_key_value_heads=w["kv_heads"], head_dim=HEAD_DIM, max_position_embeddings=131072,
                      tie_word_embeddings=False)
    torch.manual_seed(0)
    old_dtype = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = LlamaForCausalLM(cfg).eval()
    finally:
        torch.set_default_dtype(old_dtype)
    shard = HeadShard.from_process_group() if world > 1 else HeadShard()
    gen = torch.Generator(device=dev).manual_seed(99)
    B, N = w["batch"], w["context"]
    layers = []
    with torch.inference_mode():
        for _ in range(w["layers"]):
            k = synth_on_device(torch, (B, w["kv_heads"], N, HEAD_DIM), gen, torch.bfloat16)
            v = synth_on_device(torch, (B, w["kv_heads"], N, HEAD_DIM), gen, torch.bfloat16)
            layer = PackedMSELayer(bits=w["bits"], use_qjl_keys=w["use_qjl"], quantize_decode=True,
                                   reserve_tokens=steps + warmup + 8, shard=shard)
            layer.initialize_from_dense(k, v)
            layers.append(layer)
            del k, v
        cache = Cache(layers=layers)
        old_impl = enable_turboquant_attention(model, cache)
        first = torch.randint(0, w["vocab"], (B, 1), device=dev, generator=gen)
        sampler = ClockSampler(local_rank)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        def fence():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        try:
            q_heads = w["q_heads"]
            if all(layer.supports_static_decode(q_heads) for layer in layers):
                # (sharded layers exchange their outputs through the fused peer gather inside the step)
                with RecordedDecoder(model, cache, first, warmup + steps) as dec:
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
    if rank == 0:
        unit = bytes_per_unit(w["bits"], w["use_qjl"])
        packed_bytes = unit * B * w["kv_heads"] * N * w["layers"]
        weight_bytes = sum(p.numel() * p.element_size() for p in model.parameters())
        line = {
            "metric": "decode_tok_per_s_32k_ctx", "value": B * 1e3 / ms, "unit": "tok/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": args.model_scaling,
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["name"], "global_batch": B, "context": N, "layers": w["layers"],
                       "q_heads": w["q_heads"], "kv_heads": w["kv_heads"], "bits": w["bits"], "mode": "Q_prod",
                       "parallelism": f"kv-head-shard{world}, weights replicated" if world > 1 else "single",
                       "decode_step": "CUDA graph replay" if recorded else "eager"},
            "packed_kv_bytes_per_step": packed_bytes, "weight_bytes": weight_bytes,
            "hbm_gbs_lower_bound": (packed_bytes / world + weight_bytes) / (ms * 1e-3) / 1e9,
            "tokens_checksum": int(tokens.sum().item()),
            "clocks": clocks,
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


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
                    help="model workload at N > 1: strong = batch 16 in total (BASELINE config 5), weak = 16 per GPU")
    ap.add_argument("--layers", type=int, default=None, help="model workload: override the layer count (smoke runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "model":
        run_model_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
