"""Benchmark of the hot path: one routed-MoE decode layer, batch 1 (config 1).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one pass of the layer over one token: router (384 experts, top-8), the 8
selected INT4 experts, the bf16 shared expert, weighted combine.  Weights are
synthetic (seeded) with the shapes and distributions of the configuration; no
dataset or checkpoint is involved.  Prints ONE JSON line on rank 0.

  value      layer-tokens/s with inputs resident in HBM (device-timed, CUDA events)
  e2e        the same through the host-buffer C-ABI call (pinned host x in, y out,
             both copies and the synchronisation inside the timed region)
  roofline   algorithmic bytes per layer pass / device time, against the measured
             HBM copy bandwidth of this pool (MEASURED_PEAKS.json)
  cpu_baseline  the CPU oracle (a port of the reference arithmetic) on the host cores

--impl reference times the reference arithmetic on the host cores (the reference's
GPU executor cannot run without its storage stack; its math is restated in oracle/).

Between steps the layer is rotated over several distinct synthetic layers and the
token over a pool of inputs, so that the weights read by a step (292 MB) were last
touched several hundred MB ago: nothing is served from L2 across steps.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode tok/s, INT4 MoE layer (batch 1)"
WORKLOAD = "config 1: routed-MoE decode layer, batch 1, 384 INT4 experts top-8 + bf16 shared expert, hidden 7168"
HBM_FALLBACK_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the decode kernel (ncu capture of a 64-expert layer; a
# launch reads 8 experts whatever the expert count): 289.5 MB read + 8.8 MB written
NCU_TRAFFIC_BYTES_PER_LAUNCH = 298.3e6


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return HBM_FALLBACK_GBS, "fallback"


def tensor_roofline(flops, ms_per_step):
    """For the batched layer: the same step against the measured dense bf16 throughput (sustained figure)."""
    if not flops:
        return {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            tf, kind = float(json.load(f)["bf16_tflops_sustained"]), "measured"
    except Exception:
        tf, kind = 1400.0, "fallback"
    got = flops / (ms_per_step * 1e-3) / 1e12
    return {"roofline_tensor": {"bound": "tensor", "achieved": got, "peak": tf, "unit": "TFLOP/s", "frac": got / tf,
                                "peak_kind": kind}}


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 6:
                    continue
                try:
                    sm.append(float(parts[0]))
                    mx = max(mx, float(parts[1]))
                except ValueError:
                    continue
                for n, v in zip(names, parts[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.unlink(self.path)
        except Exception:
            pass
        if not sm:  # the sampler produced nothing (a very short run): one reading taken now, marked as such
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=10).stdout.strip().splitlines()[0]
                parts = [p.strip() for p in out.split(",")]
                return {"sm_mhz": float(parts[0]), "sm_max_mhz": float(parts[1]),
                        "reasons": [n for n, v in zip(names, parts[2:6]) if v.lower().startswith("active")], "samples": 0,
                        "note": "read once after the timed region"}
            except Exception:
                return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "note": "nvidia-smi gave no reading"}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def host_layer_for_oracle(w, token_ids):
    """Host copies of what the oracle needs for the given routed experts."""
    import numpy as np
    import torch
    chosen = sorted(set(int(e) for e in token_ids))
    experts = w["router_w"].shape[0]
    slot_of = np.full(experts, -1, np.int32)
    for i, e in enumerate(chosen):
        slot_of[e] = i
    idx = torch.tensor(chosen, device=w["gate_w"].device)

    def bits(t):
        return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)

    def words(t):
        return t.detach().contiguous().cpu().numpy().view(np.uint32)

    h = dict(slot_of=slot_of, router_w=bits(w["router_w"]), router_bias=w["router_bias"].float().cpu().numpy())
    for k in ("gate_w", "up_w", "down_w"):
        h[k] = words(w[k].index_select(0, idx))
    for k in ("gate_s", "up_s", "down_s"):
        h[k] = bits(w[k].index_select(0, idx))
    for k in ("shared_gate", "shared_up", "shared_down"):
        h[k] = bits(w[k])
    return h


def oracle_layer_token(orc, h, x_f32):
    out, _, _ = orc.moe_layer(h["router_w"], h["router_bias"], h["slot_of"], h["gate_w"], h["gate_s"], h["up_w"], h["up_s"],
                              h["down_w"], h["down_s"], h["shared_gate"], h["shared_up"], h["shared_down"], x_f32,
                              mode=orc.REF_EXACT)
    return out


def decode_config(world, n_layers, pool, experts=384):
    """The `config` object of the headline line; both arms print the same one."""
    from blok_b200 import synth
    return {"workload": WORKLOAD if experts == 384 else "REDUCED CASE (%d experts, profiler capture size) of " % experts + WORKLOAD,
            "parallelism": "1 GPU" if world == 1 else "replicas x%d" % world,
            "l2": "rotating %d distinct layers and %d tokens; a step's 292 MB were last read > L2 capacity ago" % (n_layers, pool),
            "algorithmic_bytes_per_step": synth.moe_layer_bytes()}


def cpu_arm(steps, warmup, device):
    """Times the reference arithmetic (oracle port, all host threads) on `steps` layer-tokens of config 1."""
    import numpy as np
    import torch
    from blok_b200 import synth
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle as orc
    # torchrun exports OMP_NUM_THREADS=1 to its ranks; the CPU arm is meant to use every core this process may run on
    orc.set_num_threads(len(os.sched_getaffinity(0)))
    # Weights are drawn with the same generator as the GPU arm; only the experts the sampled tokens route to are
    # brought to the host (the full layer is 9.5 GB).
    w = synth.moe_layer_weights(device, seed=1)
    xs = synth.activations(max(steps + warmup, 1), 7168, device, 1).float().cpu().numpy()
    ids, _, _, _ = orc.router(w["router_w"].view(torch.int16).cpu().numpy().view(np.uint16),
                              w["router_bias"].float().cpu().numpy(), xs, mode=orc.REF_EXACT)
    h = host_layer_for_oracle(w, ids.ravel())
    del w
    for i in range(warmup):
        oracle_layer_token(orc, h, xs[i:i + 1])
    t0 = time.perf_counter()
    for i in range(warmup, warmup + steps):
        oracle_layer_token(orc, h, xs[i:i + 1])
    dt = time.perf_counter() - t0
    return steps / dt, dt, orc.num_threads()


def ep_parity_check(rank, world, device, comm):
    """A reduced layer through the expert-parallel path on every rank against the single-GPU batched layer on the rank's
    own tokens, with one GEMM implementation forced at a time (the same kernel then computes every row on both sides):
    the outputs must be bit-equal.  Returns (ok on every rank, worst absolute difference over the ranks)."""
    import torch
    import torch.distributed as dist
    from blok_b200 import lib, synth
    hidden, inter, experts, shared = 1024, 512, 128, 512
    w = synth.moe_layer_weights(device, seed=77, hidden=hidden, inter=inter, experts=experts, shared_inter=shared)
    for k in ("gate_s", "up_s", "down_s"):
        w[k] = (w[k].float() * 8).bfloat16()
    w["router_w"] = (w["router_w"].float() * 20).bfloat16()
    per = experts // world
    shard = dict(w)
    for k in ("gate_w", "gate_s", "up_w", "up_s", "down_w", "down_s"):
        shard[k] = w[k][rank * per:(rank + 1) * per].contiguous()
    layer = lib.MoeEp(comm, shard, max_tokens=64)
    full = lib.MoeLayer(w, max_tokens=64)
    ok, worst = True, 0.0
    old = os.environ.get("BLOK_WGEMM_IMPL")
    for step, impl in enumerate(("mma", "tc")):
        os.environ["BLOK_WGEMM_IMPL"] = impl
        x = synth.activations(24 + 5 * rank, hidden, device, 900 + rank + 10 * step)
        y, ids, wts = layer.forward(x, return_routing=True)
        layer.check()
        ref, rid, rw = full.batched(x, return_routing=True)
        ok = ok and torch.equal(ids, rid) and torch.equal(wts, rw) and torch.equal(y, ref)
        worst = max(worst, float((y.float() - ref.float()).abs().max()))
    if old is None:
        del os.environ["BLOK_WGEMM_IMPL"]
    else:
        os.environ["BLOK_WGEMM_IMPL"] = old
    flag = torch.tensor([0.0 if ok else 1.0, worst], device=device)
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    layer.close()
    full.close()
    return float(flag[0]) == 0.0, float(flag[1])


def ep_measure(T, rank, world, device, comm, steps, warmup, experts=384):
    """Config 2 at T tokens with the experts split over the ranks (blok_moe_ep_*): per-pass device time (max over the
    ranks), this rank-set's roofline figures (the slowest rank's bytes), the exchange volume and the phase times."""
    import torch
    import torch.distributed as dist
    from blok_b200 import lib, synth
    Tl = T // world
    per = experts // world
    nl = 2 if experts == 384 else 1
    reps = []
    for i in range(nl):
        w = synth.moe_layer_weights(device, seed=2 + 31 * i, experts=experts)
        if world > 1:
            for k in ("gate_w", "gate_s", "up_w", "up_s", "down_w", "down_s"):
                w[k] = w[k][rank * per:(rank + 1) * per].contiguous()
            torch.cuda.empty_cache()
        reps.append(lib.MoeEp(comm, w, max_tokens=max(Tl, 1)))
    xs = [synth.activations(Tl, 7168, device, 2 + 7 * i + rank) for i in range(4)]
    outs = torch.empty((Tl, 7168), dtype=torch.bfloat16, device=device)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for i in range(max(warmup, 3)):
            reps[i % nl].forward(xs[i % 4], out=outs)
        barrier()
        l0 = lib.kernel_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            reps[i % nl].forward(xs[i % 4], out=outs)
        e1.record()
        barrier()
        launches = lib.kernel_launch_count() - l0
        for r in reps:
            r.check()
        # one more pass of layer 0 on input 0 with the phase events on, and its routing for the byte counts
        reps[0].profile(True)
        _, ids, _ = reps[0].forward(xs[0], out=outs, return_routing=True)
        phases = reps[0].phase_ms()
        stats = reps[0].stats()
        reps[0].profile(False)
        torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=device)
    # distinct experts of THIS rank that the whole batch routes to (every rank's ids gathered)
    ids32 = (ids.view(torch.int16).to(torch.int32) & 0xFFFF).contiguous()      # NCCL carries no 16-bit integers
    ids_all = [torch.empty_like(ids32) for _ in range(world)] if world > 1 else [ids32]
    if world > 1:
        dist.all_gather(ids_all, ids32)
    flat = torch.cat([t.long().view(-1) for t in ids_all])
    mine = flat[(flat >= rank * per) & (flat < (rank + 1) * per)].unique()
    fig = torch.tensor([float(mine.numel()), float(stats["received"]), float(stats["remote"]), phases["route"], phases["dispatch"],
                        phases["shared"], phases["wait_rows"], phases["experts"], phases["combine"]], device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(fig, op=dist.ReduceOp.MAX)
    per_step = float(ms.item()) / steps
    distinct, received, remote = int(fig[0]), int(fig[1]), int(fig[2])
    alg = distinct * 24772608 + 5505024 + 88080384 + 4 * Tl * 7168 + 2 * received * 7168 * 2   # the busiest rank
    flops = 2.0 * (received * 3 * 7168 * 2048 + Tl * (3 * 7168 * 2048 + 7168 * experts))
    peak, peak_kind = measured_peak()
    rec = {"T": T, "parallelism": "expert parallel x%d" % world if world > 1 else "1 GPU, through the same exchange kernels",
           "ms_per_pass": per_step, "tok_per_s": T / (per_step * 1e-3),
           "experts_per_gpu": per, "distinct_experts_busiest_gpu": distinct, "rows_received_busiest_gpu": received,
           "remote_assignments_busiest_gpu": remote, "exchange_bytes_each_way_busiest_gpu": remote * 7168 * 2,
           "roofline": {"bound": "hbm", "achieved": alg / (per_step * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                        "frac": alg / (per_step * 1e-3) / 1e9 / peak, "peak_kind": peak_kind, "bytes_busiest_gpu": alg},
           "phase_ms_max_over_ranks": {k: float(fig[3 + i]) for i, k in enumerate(("route", "dispatch", "shared", "wait_rows",
                                                                                  "experts", "combine"))},
           "launches_per_pass": launches / steps, **tensor_roofline(flops, per_step)}
    for r in reps:
        r.close()
    del reps
    torch.cuda.empty_cache()
    return rec, launches


def other_workload(a, rank, world, device, steps, warmup):
    """Configs 2 and 3 through the same timing rules (CUDA events, barrier both sides, max over ranks)."""
    import torch
    import torch.distributed as dist
    from blok_b200 import lib, synth

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    peak, peak_kind = measured_peak()
    flops = None  # set by the batched workloads: multiply-add work of a step on this GPU
    extra = {}    # workload-specific figures that go into the line's config
    unit = "tok/s"
    if a.workload == "model":
        # config 4 on what ONE GPU holds: layer 0 dense + (model_layers - 1) MoE layers of the full shapes, full
        # vocabulary, batch 1, greedy decode after a 32-token prompt replay.  A step is one new token through every
        # layer (embedding, MLA, dense / MoE, final norm, lm_head, argmax); a step reads > 6 GB, far beyond L2.
        L, B = a.model_layers, a.batch
        model = lib.Model(seed=4 + rank, layers=L, max_batch=B, max_ctx=max(256, 64 + steps + warmup + 8))
        ids = torch.randint(0, 163840, (B,), device=device, dtype=torch.int32)
        for _ in range(32):
            ids = model.step(ids)
        state = {"ids": ids}

        def run(i):
            state["ids"] = model.step(state["ids"])
        moe_bytes = 291767808 + 202244096          # routed-MoE decode layer + MLA projections, per MoE layer
        dense_bytes = 3 * 18432 * 7168 * 2 + 202244096
        # batch 1: 8 experts per layer; a batch touches more (counted as B x 8 distinct, an upper bound, capped at 384)
        moe_bytes += (min(384, 8 * B) - 8) * 24772608
        alg = (L - 1) * moe_bytes + dense_bytes + 163840 * 7168 * 2   # + lm_head; the cache (<= 300 tokens) is negligible
        unit_tokens = world * B
        workload = ("config 4 on one GPU: %d of the 61 layers (1 dense + %d MoE, full shapes), vocab 163840, batch %d, "
                    "greedy decode%s" % (L, L - 1, B, "" if world == 1 else ", replicas x%d" % world))
        scaling = "weak"
        metric = "decode tok/s, %d-layer model (batch %d)" % (L, B)
    elif a.workload == "prefill512":
        # config 4's prompt on what ONE GPU holds: 512 random ids through the first model_layers layers in chunks of 64
        # tokens (blok_model_prefill); a step is the whole prompt and samples its last token.  The reference replays the
        # prompt token by token (src/kimi_exec.cu:885-886); `--workload model` times that form per token.
        L, P, chunk = a.model_layers, 512, 64
        model = lib.Model(seed=4 + rank, layers=L, max_batch=1, max_ctx=P + 8, prefill_chunk=chunk)
        prompts = [torch.randint(0, 163840, (P,), device=device, dtype=torch.int32) for _ in range(4)]

        def run(i):
            # reset clears the positions on the default stream: fence it against the prompt on the timing stream
            torch.cuda.synchronize()
            model.reset()
            torch.cuda.synchronize()
            model.prefill(prompts[i % 4])
        # per chunk and MoE layer: attention weights once per 8 tokens, the experts the chunk routes to once (at most
        # 64 x 8 distinct, capped at 384), router and shared expert once; the dense layer once per 5 tokens
        per_chunk = (L - 1) * (202244096 * (chunk // 8) + 384 * 24772608 + 5505024 + 88080384) + \
            (3 * 18432 * 7168 * 2) * ((chunk + 4) // 5) + 202244096 * (chunk // 8)
        alg = per_chunk * (P // chunk) + 163840 * 7168 * 2
        unit_tokens = world * P
        workload = ("config 4's 512-token prompt on one GPU: %d of the 61 layers (1 dense + %d MoE, full shapes), chunks of %d "
                    "tokens, last token sampled%s" % (L, L - 1, chunk, "" if world == 1 else ", replicas x%d" % world))
        scaling = "weak"
        metric = "prefill tok/s, %d-layer model (512-token prompt)" % L
    elif a.workload == "model61":
        # config 4: the 61-layer model sharded expert-parallel over the ranks (384 / world experts per GPU, attention,
        # router, shared expert, embedding and lm_head replicated), batch 1, greedy decode after a 16-token prompt replay.
        # With fewer than 8 GPUs only as many layers as fit are built, and the line says how many.
        B = a.batch
        per_layer = 9.513e9 / world + 0.32e9
        L = a.model_layers if a.model_layers != 12 else min(61, int(140e9 // per_layer))
        comm = lib.Comm() if world > 1 else None
        model = lib.Model(seed=4, layers=L, max_batch=B, max_ctx=max(256, 32 + steps + warmup + 8), ep_rank=rank, ep_world=world)
        if comm is not None:
            model.set_comm(comm)
        state = {"ids": torch.randint(0, 163840, (B,), device=device, dtype=torch.int32)}
        if world > 1:
            dist.broadcast(state["ids"], 0)

        def run(i):
            state["ids"] = model.step(state["ids"])
        prompt_side = torch.cuda.Stream()
        with torch.cuda.stream(prompt_side):
            for _ in range(16):
                run(0)
        torch.cuda.synchronize()
        model.check()
        # every rank must hold the same next ids: the layers are the same arithmetic on every rank after the all-reduce
        if world > 1:
            both = [torch.empty_like(state["ids"]) for _ in range(world)]
            dist.all_gather(both, state["ids"])
            if any(not torch.equal(both[0], t) for t in both):
                if rank == 0:
                    print(json.dumps({"error": "sharded model: ranks disagree on the next token"}))
                return 3
        # per GPU and step: the replicated weights once, and this GPU's share of the experts the batch routes to (B x 8
        # distinct at most, capped at 384, spread evenly over the ranks)
        alg = (L - 1) * (202244096 + 5505024 + 88080384 + min(384, 8 * B) * 24772608 / world) + \
            (3 * 18432 * 7168 * 2 + 202244096) + 163840 * 7168 * 2
        unit_tokens = B
        workload = ("config 4: %d-layer model (1 dense + %d MoE layers, full shapes, vocab 163840), batch %d, greedy decode, "
                    "experts split over %d GPU(s), one all-reduce per MoE layer" % (L, L - 1, B, world))
        scaling = "strong"
        metric = "decode tok/s, %d-layer model (batch %d)" % (L, B)
    elif a.workload.startswith("batched"):
        T = int(a.workload[len("batched"):])
        if world > 1:
            comm = lib.Comm()
            ok, worst = ep_parity_check(rank, world, device, comm)
            if not ok:
                if rank == 0:
                    print(json.dumps({"error": "expert-parallel parity check failed", "worst_abs_diff": worst}))
                return 3
            sampler = ClockSampler(device.index or 0)
            if rank == 0:
                sampler.start()
            rec, launches = ep_measure(T, rank, world, device, comm, steps, warmup, a.experts)
            clocks = sampler.stop() if rank == 0 else None
            if rank == 0:
                print(json.dumps({
                    "metric": "tok/s, INT4 MoE layer (T=%d)" % T, "value": rec["tok_per_s"], "unit": "tok/s", "n_gpus": world,
                    "steps": steps, "warmup": warmup, "ms_per_step": rec["ms_per_pass"], "higher_is_better": True,
                    "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                    "config": {"workload": "config 2: batched routed-MoE layer, T=%d tokens, expert parallel x%d (%d experts per "
                                           "GPU), dispatch/combine in the library's kernels over NVLink peer memory" %
                                           (T, world, a.experts // world),
                               "l2": "two layers and four inputs rotated", "ep_parity": "bit-equal to the single-GPU layer"},
                    "roofline": rec["roofline"], "roofline_tensor": rec.get("roofline_tensor"), "ep": rec,
                    "gpu_launches": int(launches), "clocks": clocks}))
            comm.close()
            dist.destroy_process_group()
            return 0
        nl = 2 if a.experts == 384 else 1  # a reduced case (profiler capture) holds one layer
        reps = [lib.MoeLayer(synth.moe_layer_weights(device, seed=2 + 31 * i, experts=a.experts), max_tokens=max(T, 2))
                for i in range(nl)]
        xs = [synth.activations(T, 7168, device, 2 + 7 * i + rank) for i in range(4)]
        run = lambda i: reps[i % nl].batched(xs[i % 4])
        ids = lib.router(reps[0].weights["router_w"], reps[0].weights["router_bias"], xs[0])[0]
        distinct = int((ids.view(torch.int16).long() & 0xFFFF).unique().numel())
        alg = distinct * 24772608 + 5505024 + 88080384 + 4 * T * 7168
        unit_tokens = T
        # multiply-adds of the pass: T x 8 assignments through three 7168 x 2048 matrices, the tokens through the shared
        # expert and the router
        flops = 2.0 * (T * 8 * 3 * 7168 * 2048 + T * (3 * 7168 * 2048 + 7168 * a.experts))
        workload = "config 2: batched routed-MoE layer, T=%d tokens, 1 GPU" % T
        if a.experts != 384:
            workload = "REDUCED CASE (%d experts, profiler capture size) of " % a.experts + workload
        scaling = "strong"
        metric = "tok/s, INT4 MoE layer (T=%d)" % T
    elif a.workload == "expert":
        # config 0: ONE routed expert's SwiGLU FFN at batch 1 (blok_expert_ffn: two launches, gate/up with the SiLU*up
        # epilogue and down).  A step runs 16 experts back to back out of 48 rotated ones (1.19 GB, so an expert's 24.8 MB
        # were last read 1.17 GB ago); per-expert time = step / 16.  The cold latency of a single call (L2 flushed by a
        # 512 MB write, one expert, events around it) is measured before the timed loop and reported beside it.
        NE = 48
        g = torch.Generator(device=device).manual_seed(20 + rank)
        ew = synth.expert_weights(NE, 7168, 2048, g, device)
        xv = synth.activations(1, 7168, device, 0).view(-1).contiguous()
        ws = torch.empty(lib.load().blok_expert_ffn_workspace_bytes(7168, 2048), dtype=torch.uint8, device=device)
        one = lambda e: lib.expert_ffn(ew["gate_w"][e], ew["gate_s"][e], ew["up_w"][e], ew["up_s"][e], ew["down_w"][e],
                                       ew["down_s"][e], xv, workspace=ws)

        def run(i):
            for k in range(16):
                one((16 * i + k) % NE)
        flush = torch.empty(512 << 20, dtype=torch.uint8, device=device)
        cold = []
        for r in range(8):
            flush.fill_(r)
            c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            c0.record()
            one(r)
            c1.record()
            torch.cuda.synchronize()
            cold.append(c0.elapsed_time(c1) * 1e3)
        del flush
        cold.sort()
        extra["cold_single_expert_us"] = {"median": cold[len(cold) // 2], "min": cold[0], "samples": len(cold)}
        extra["experts_per_step"] = 16
        alg = 16 * 24772608 + 16 * 2 * 7168 * 2
        unit_tokens = 16 * world
        workload = ("config 0: single routed expert SwiGLU FFN, batch 1, 16 experts per step out of 48 rotated (1.19 GB)%s"
                    % ("" if world == 1 else ", replicas x%d" % world))
        scaling = "weak"
        metric = "expert FFNs/s, INT4 W4A16 (batch 1)"
        unit = "experts/s"
    elif a.workload == "gemv":
        # config 0's building block at a size the launch rate does not bound: one INT4 mat-vec y = W x (matvec_i4_slice,
        # src/kimi_exec.cu:688) over 32 experts' gate matrices stacked, [65536, 7168] = 264 MB per call, 3 such matrices
        # rotated.  BLOK_I4_GEMV_IMPL=imma in the environment times the integer tensor-core consumer instead of the
        # bf16-operand one.
        R = 65536
        g = torch.Generator(device=device).manual_seed(11 + rank)
        mats = [(torch.randint(-2 ** 31, 2 ** 31 - 1, (R, 896), generator=g, device=device, dtype=torch.int32),
                 (torch.randn((R, 224), generator=g, device=device) * 0.003).abs().bfloat16()) for _ in range(3)]
        xv = synth.activations(1, 7168, device, 5).view(-1).contiguous()
        run = lambda i: lib.i4_gemv(mats[i % 3][0], mats[i % 3][1], xv)
        alg = R * 896 * 4 + R * 224 * 2 + 7168 * 2 + R * 2
        unit_tokens = world
        workload = ("config 0 building block: INT4 mat-vec [%d x 7168] (32 gate matrices stacked), batch 1, impl=%s%s" %
                    (R, os.environ.get("BLOK_I4_GEMV_IMPL", "bf16-operand"), "" if world == 1 else ", replicas x%d" % world))
        scaling = "weak"
        metric = "mat-vecs/s, INT4 [%d x 7168]" % R
        unit = "mat-vecs/s"
    else:
        ctx = int(a.workload[len("mla"):])
        B = 8 if a.batch == 1 else min(a.batch, 64)   # config 3 is batch 8; --batch N measures the block at N sequences
        layer = lib.MlaLayer(synth.mla_weights(device, seed=3), yarn_factor=32.0, max_batch=max(B, 8), max_ctx=ctx + 8)
        ncache = 6 if ctx <= 4096 and B <= 8 else 3
        caches = [synth.latent_cache(B, ctx + 8, device, seed=10 + i + rank) for i in range(ncache)]
        n = synth.activations(B, 7168, device, 3)
        ctx_len = torch.full((B,), ctx, dtype=torch.int32, device=device)
        out = torch.empty((B, 7168), dtype=torch.bfloat16, device=device)
        run = lambda i: layer.decode(n, caches[i % ncache], ctx_len, out=out)
        alg = B * ctx * 1152 + 202244096
        unit_tokens = B * world
        workload = "config 3: MLA absorbed decode block, batch %d, ctx %d, bf16 latent cache%s" % (B, ctx, "" if world == 1 else ", replicas x%d" % world)
        scaling = "weak"
        metric = "tok/s, MLA decode block (batch %d, ctx %d)" % (B, ctx)
    # a side stream: the whole-model step replays a CUDA graph, which the legacy default stream cannot capture
    side = torch.cuda.Stream()
    torch.cuda.synchronize()
    sampler = ClockSampler(device.index or 0)
    if rank == 0:
        sampler.start()      # before the warm-up, so that a short timed region still has samples under load
    with torch.cuda.stream(side):
        for i in range(max(warmup, 3)):
            run(i)
        barrier()
        l0 = lib.kernel_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            run(warmup + i)
        e1.record()
        barrier()
    launches = lib.kernel_launch_count() - l0
    clocks = sampler.stop() if rank == 0 else None
    ms = torch.tensor([e0.elapsed_time(e1)], device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    if rank == 0:
        per_step = ms / steps
        achieved = alg / (per_step * 1e-3) / 1e9
        print(json.dumps({
            "metric": metric, "value": unit_tokens * steps / (ms / 1e3), "unit": unit, "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": per_step, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload, "algorithmic_bytes_per_step_per_gpu": alg,
                       "l2": "weights and caches rotated over several copies larger than L2", **extra},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "traffic": None},
            **tensor_roofline(flops, per_step),
            "gpu_launches": int(launches), "clocks": clocks}))
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=3, help="distinct synthetic layers rotated between steps")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=1, help="sequences per step of the `model` workloads (up to 64); with mla*: sequences of the block instead of config 3's 8")
    ap.add_argument("--model-layers", type=int, default=12, help="layers of the `model` workload (one GPU holds about 15)")
    ap.add_argument("--experts", type=int, default=384,
                    help="routed experts per layer; below 384 the run is a reduced case for profiler captures, "
                         "not the benchmark configuration, and the line says so")
    ap.add_argument("--workload", default="decode", choices=["decode", "expert", "batched64", "batched2048", "mla4096", "mla32768", "model", "model61", "prefill512", "gemv"],
                    help="decode = config 1 (the default, the headline metric); batched* = config 2 (expert parallel "
                         "when --gpus > 1); mla* = config 3 (attention block, batch 8)")
    a = ap.parse_args()

    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if a.impl == "reference":
        if rank != 0:
            return 0
        steps = a.steps if a.steps is not None else 12
        warmup = a.warmup if a.warmup is not None else 3
        steps_run = min(steps, 64)  # bounded sample: each step is one full layer-token on the host cores
        device = torch.device("cuda:0") if torch.cuda.is_available() else torch.device("cpu")
        rate, dt, threads = cpu_arm(steps_run, min(warmup, 3), device)
        line = {"impl": "reference", "metric": METRIC, "value": rate, "unit": "tok/s", "n_gpus": a.gpus, "steps": steps,
                "warmup": warmup, "ms_per_step": 1e3 / rate, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": decode_config(a.gpus, a.layers, 64),
                "note": "reference arithmetic on host cores (oracle port); the reference's GPU executor needs its NVMe/uGDS "
                        "storage stack and cannot run",
                "cpu_baseline": {"value": rate, "unit": "tok/s", "cores": threads, "kind": "port",
                                 "sample": "%d layer-tokens of config 1 (%.1f s)" % (steps_run, dt)},
                "e2e": {"value": rate, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return 0

    steps = a.steps if a.steps is not None else 4000
    warmup = a.warmup if a.warmup is not None else 50
    import torch.distributed as dist
    from blok_b200 import lib, synth
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    lib.load()
    if a.workload != "decode":
        return other_workload(a, rank, world, device, steps if a.steps is not None else 20, warmup if a.warmup is not None else 5)

    # distinct layers (each 9.5 GB of packed experts + its own router and shared expert)
    layers = [lib.MoeLayer(synth.moe_layer_weights(device, seed=1 + 17 * i + 1000 * rank, experts=a.experts))
              for i in range(a.layers)]
    pool = 64
    xs = synth.activations(pool, 7168, device, 1 + rank)
    y = torch.empty(7168, dtype=torch.bfloat16, device=device)

    def step(i):
        layers[i % len(layers)].decode(xs[i % pool], out=y)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()      # before the warm-up, so that a short timed region still has samples under load
    for i in range(max(warmup, 3)):
        step(i)
    barrier()
    l0 = lib.kernel_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(warmup + i)
    e1.record()
    barrier()
    launches = lib.kernel_launch_count() - l0
    ms = torch.tensor([e0.elapsed_time(e1)], device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    clocks = sampler.stop() if rank == 0 else None

    # end to end through the host-buffer C-ABI call
    xh = xs.cpu().pin_memory()
    yh = torch.empty(7168, dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(min(steps // 2, 1000), 1)
    for i in range(5):
        layers[i % len(layers)].decode_host(xh[i % pool], yh)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for i in range(e2e_steps):
        layers[i % len(layers)].decode_host(xh[i % pool], yh)
    f1.record()
    barrier()
    e2e_ms = torch.tensor([f0.elapsed_time(f1)], device=device)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e_ms.item())

    # N > 1: the sharded path of the same layer type (config 2, expert parallel) measured in the same run
    ep_rec = None
    if world > 1:
        for L in layers:
            L.close()
        del layers
        torch.cuda.empty_cache()
        comm = lib.Comm()
        ok, worst = ep_parity_check(rank, world, device, comm)
        if not ok:
            if rank == 0:
                print(json.dumps({"error": "expert-parallel parity check failed", "worst_abs_diff": worst}))
            return 3
        ep_rec = {"parity": "bit-equal to the single-GPU batched layer on every rank (reduced layer, both GEMM kernels)"}
        for T in (2048, 64):
            ep_rec["T%d" % T], _ = ep_measure(T, rank, world, device, comm, 20, 5)
        comm.close()
        layers = []

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0

    ms_per_step = ms / steps
    value = world * steps / (ms / 1e3)
    peak, peak_kind = measured_peak()
    alg_bytes = synth.moe_layer_bytes()
    achieved = alg_bytes / (ms_per_step * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": decode_config(world, a.layers, pool, a.experts),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": peak_kind, "frac_of_nominal_8TBs": achieved / 8000.0,
                     "kernel": "moe decode layer (%d launches per step)" % round(launches / steps),
                     "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH},
        "e2e": {"value": world * e2e_steps / (e2e_ms / 1e3), "unit": "tok/s", "h2d_bytes_per_step": 7168 * 2,
                "d2h_bytes_per_step": 7168 * 2, "ms_per_step": e2e_ms / e2e_steps},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    if ep_rec is not None:
        line["ep"] = ep_rec
    if world == 1 and not a.no_cpu_baseline:
        for L in layers:
            L.close()
        del layers
        torch.cuda.empty_cache()
        rate, dt, threads = cpu_arm(48, 1, device)
        line["cpu_baseline"] = {"value": rate, "unit": "tok/s", "cores": threads, "kind": "port",
                                "sample": "48 layer-tokens of config 1 (%.1f s)" % dt}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
