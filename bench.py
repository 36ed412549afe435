"""Decode throughput of the Qwen3-30B-A3B-shape MoE on the B200 kernels.

    python bench.py --gpus N --steps K --warmup W            # our arm
    python bench.py --impl reference --gpus N --steps K --warmup W   # CPU reference arm

Workload (BASELINE.json configs[3]): 48 layers, hidden 2048, 32 q / 4 kv heads, head_dim 128,
128 experts top-8 (renormalised softmax routing), expert FFN 768, vocab 151936; random init
N(0, 0.02) bf16; decode at batch 512 with a 2048-token paged context (16-token pages, page
table = seeded random permutation).  A "step" is one decode step of one 512-sequence batch:
embedding -> 48 decoder layers -> final norm -> lm_head -> greedy token + its logprob.
With N > 1 GPUs the layers are split evenly over N pipeline stages and N batches are in
flight (one per stage).  Every hand-off goes through the library's PPMessager
(send_gen_ctx / recv_gen_ctx / send_infer_out / recv_infer_out): hidden states AND the step's
metadata (positions, slot mapping, query_start_loc, context lengths, block-table deltas) travel
every step, nothing is pre-resident on later stages.  Per-GPU work is fixed, so scaling is
"weak" and a step advances all N in-flight batches by one token.  The pipeline is kept full
across the timed region: warm-up steps run straight into the timed ones and each rank times
its own K steps with CUDA events (max over ranks).

Prints ONE JSON line (rank 0).  `value` is device-timed with inputs resident in HBM;
`e2e` uploads each step's per-request counters from pinned host memory, builds the step's input
buffers from them on the device (b200_prepare_step; block tables and the previous step's tokens
stay in HBM) and reads tokens/logprobs back.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "decode_tokens_per_s"
UNIT = "tokens/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    # development overrides (the default is the BASELINE workload)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--batch", type=int, default=512)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--quick", action="store_true", help="device-timed run only (for profiler captures)")
    ap.add_argument("--model", default="qwen3-30b-a3b-shape",
                    help="another preset (qwen3-1.7b-shape, qwen2-1.5b-shape, moonlight-16b-a3b-shape) runs a "
                         "one-GPU decode step of that shape as a side measurement with its own JSON line")
    ap.add_argument("--prefill-chunk", type=int, default=0, metavar="TOKENS",
                    help="side measurement: one chunked-prefill step of TOKENS prompt tokens after --ctx cached ones")
    ap.add_argument("--ragged-attention", action="store_true",
                    help="side measurement: decode attention over a ragged batch, with / without sequence order")
    ap.add_argument("--unfused-head", action="store_true",
                    help="materialise the [batch, vocab] logits and select tokens with a second kernel")
    ap.add_argument("--skew", action="store_true",
                    help="side measurement: one MoE layer of the model with near-uniform routing and with a "
                         "Zipf(1.1) router bias: rows per expert, token tiles, fc1 / fc2 time")
    ap.add_argument("--row-kernels", action="store_true",
                    help="side measurement: the row kernels (RMSNorm, log_softmax, gather_logprob, kv_store) at the "
                         "operator-suite shapes, rotating over inputs larger than L2, GB/s per kernel")
    ap.add_argument("--train-kernels", action="store_true",
                    help="side measurement: forward + backward of the packed attention call and of one fused-MoE "
                         "layer at the model's widths (the training-side operators; correctness-first kernels)")
    ap.add_argument("--prefill-attention", type=int, default=0, metavar="QLEN",
                    help="side measurement: time one causal prefill attention call of QLEN queries on the "
                         "model's head shape (context --ctx if larger) and print its own JSON line")
    return ap.parse_args()


def workload_name(args, shape):
    return (f"{shape.name} decode, batch {args.batch}, ctx {args.ctx}, page {args.page}, "
            f"{shape.num_layers} layers")


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def wait_first_sample(self, limit_s: float = 5.0):
        t0 = time.time()
        while self.proc is not None and time.time() - t0 < limit_s:
            try:
                if os.path.getsize(self.path) > 0:
                    return
            except OSError:
                return
            time.sleep(0.05)

    def mark(self) -> int:
        """Number of samples written so far (to cut the timed region out of the log)."""
        try:
            return sum(1 for _ in open(self.path))
        except Exception:
            return 0

    def stop(self, first: int = 0):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            rows = [r.split(",") for r in open(self.path).read().strip().splitlines() if r.strip()]
            rows = rows[first:] if len(rows) > first else rows[-1:]
            sm = sorted(float(r[1]) for r in rows if len(r) >= 9)
            if sm:
                out["sm_mhz"] = sm[len(sm) // 2]
                out["sm_max_mhz"] = float(rows[0][2])
                out["power_w_max"] = max(float(r[3]) for r in rows if len(r) >= 9)
                names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
                seen = set()
                for r in rows:
                    for i, n in enumerate(names):
                        if len(r) >= 9 and r[5 + i].strip().lower().startswith("active"):
                            seen.add(n)
                out["reasons"] = sorted(seen)
                out["samples"] = len(sm)
        except Exception:
            pass
        finally:
            try:
                os.unlink(self.path)
            except OSError:
                pass
        return out


# --------------------------------------------------------------------------- CPU reference arm
class CpuSample:
    """One decoder layer + the head on CPU for `seqs` sequences of the workload.

    The per-layer time is multiplied by the layer count: layers are identical in shape and cost."""

    def __init__(self, args, shape, seqs: int, threads: int):
        torch.set_num_threads(threads)
        g = torch.Generator().manual_seed(0)
        BF = torch.bfloat16
        H, D = shape.hidden, shape.head_dim
        m = shape.moe
        self.shape, self.seqs = shape, seqs

        def rn(*s):
            t = torch.empty(*s, dtype=BF)
            t.normal_(0.0, 0.02, generator=g)
            return t

        self.lw = dict(input_norm=torch.ones(H, dtype=BF), post_norm=torch.ones(H, dtype=BF),
                       qkv=rn(shape.qkv_out, H), q_norm=torch.ones(D, dtype=BF), k_norm=torch.ones(D, dtype=BF),
                       o=rn(H, shape.num_q_heads * D), router=rn(m.num_experts, H),
                       experts_gate_up=rn(m.num_experts, 2 * m.intermediate, H),
                       experts_down=rn(m.num_experts, H, m.intermediate))
        self.final_norm, self.lm_head = torch.ones(H, dtype=BF), rn(shape.vocab, H)
        pages = (args.ctx + args.page - 1) // args.page
        nblocks = seqs * pages
        self.kc = torch.empty(nblocks, args.page, shape.num_kv_heads, D, dtype=BF).normal_(generator=g)
        self.vc = torch.empty(nblocks, args.page, shape.num_kv_heads, D, dtype=BF).normal_(generator=g)
        self.ptab = torch.randperm(nblocks, generator=g).view(seqs, pages).to(torch.int32)
        self.h = torch.empty(seqs, H, dtype=BF).normal_(generator=g)
        self.pos = torch.full((seqs,), args.ctx - 1, dtype=torch.int64)
        self.slots = (self.ptab[:, (args.ctx - 1) // args.page].long() * args.page
                      + (args.ctx - 1) % args.page).to(torch.int32)
        self.cu = torch.arange(seqs + 1, dtype=torch.int32)
        self.used = torch.full((seqs,), args.ctx, dtype=torch.int32)

    def run(self) -> float:
        """Seconds one decode step of `seqs` sequences would take (layer time x layers + head)."""
        from oracle import cpu_model

        t0 = time.perf_counter()
        h2 = cpu_model.layer_forward(self.shape, self.lw, self.h, self.pos, self.slots, self.kc, self.vc, self.cu,
                                     self.used, self.ptab)
        t1 = time.perf_counter()
        cpu_model.head_forward(self.shape, self.final_norm, self.lm_head, h2)
        t2 = time.perf_counter()
        return (t1 - t0) * self.shape.num_layers + (t2 - t1)


def run_reference(args, shape, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    seqs = min(args.batch, 128)
    sample = (f"1 of {shape.num_layers} decoder layers (time x {shape.num_layers}) + final norm/lm_head/logprob, "
              f"{seqs} of {args.batch} sequences at ctx {args.ctx}, torch CPU ops, {threads} threads")
    sam = CpuSample(args, shape, seqs, threads)
    for _ in range(args.warmup):
        sam.run()
    t_tot = 0.0
    for _ in range(args.steps):
        t_tot += sam.run()
    ms = t_tot / max(args.steps, 1) * 1e3
    value = seqs / (ms / 1e3)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(args, shape), "pipeline_stages": args.gpus},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- our arm
def build_inputs(args, shape, seed, device):
    """Pinned host inputs of one decode step and their static device copies."""
    S, ctx, page = args.batch, args.ctx, args.page
    pages = (ctx + page - 1) // page
    g = torch.Generator().manual_seed(seed)
    ptab = torch.randperm(S * pages, generator=g).view(S, pages).to(torch.int32)
    host = dict(
        input_ids=torch.randint(0, shape.vocab, (S,), generator=g),
        positions=torch.full((S,), ctx - 1, dtype=torch.int64),
        slot_mapping=(ptab[:, (ctx - 1) // page].long() * page + (ctx - 1) % page).to(torch.int32),
        query_start_loc=torch.arange(S + 1, dtype=torch.int32),
        context_lens=torch.full((S,), ctx, dtype=torch.int32),
        block_tables=ptab,
    )
    host = {k: v.pin_memory() for k, v in host.items()}
    dev = {k: v.to(device) for k, v in host.items()}
    return host, dev, S * pages


def measured_peaks() -> dict:
    """The pool's measured peaks (driver-written file), {} when absent."""
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


def recorded_traffic(kernel: str, batch: int, ctx: int, page: int):
    """DRAM bytes per launch that ncu measured for `kernel` on this workload, from the tracked summary
    next to the other profiler summaries; None when that workload was never captured."""
    try:
        for line in open(os.path.join(ROOT, "profiles", "roofline_traffic.txt")):
            if line.startswith("#") or "|" not in line:
                continue
            f = [x.strip() for x in line.split("|")]
            if len(f) == 5 and f[0] == kernel and (int(f[1]), int(f[2]), int(f[3])) == (batch, ctx, page):
                return int(f[4])
    except (OSError, ValueError):
        pass
    return None


def run_prefill_chunk(args, shape):
    """Side measurement (not the contract line): one chunked-prefill step - `--prefill-chunk` prompt
    tokens of one sequence appended to `--ctx` cached tokens - through the stage runner (eager, as a
    prefill step runs), against the tensor-core bound of its GEMMs."""
    from vexact_b200 import _lib
    from vexact_b200.inferencer import StageRunner, StageWeights, StepInputs, allocate_kv_cache

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    T, page = args.prefill_chunk, args.page
    past = args.ctx
    total = past + T
    pages = (total + page - 1) // page
    weights = StageWeights.random_init(shape, 0, 1, device=device, seed=0)
    kc, vc = allocate_kv_cache(shape, 0, shape.num_layers, pages, page, device=device, fill_std=1.0, seed=0)
    g = torch.Generator().manual_seed(3)
    table = torch.randperm(pages, generator=g).view(1, pages).to(torch.int32)
    pos = torch.arange(past, total, dtype=torch.int64)
    slots = (table[0, (pos // page)].long() * page + pos % page).to(torch.int32)
    inp = StepInputs(input_ids=torch.randint(0, shape.vocab, (T,), generator=g).to(device), hidden_in=None,
                     positions=pos.to(device), slot_mapping=slots.to(device),
                     query_start_loc=torch.tensor([0, T], dtype=torch.int32, device=device),
                     context_lens=torch.tensor([total], dtype=torch.int32, device=device),
                     block_tables=table.to(device), max_seqlen_q=T)
    runner = StageRunner(weights, kc, vc, 0, 1)
    for _ in range(max(args.warmup, 2)):
        runner.step(inp)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        runner.step(inp)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / args.steps
    s = shape
    per_layer = 2.0 * T * s.hidden * (s.qkv_out + s.num_q_heads * s.v_dim)          # qkv + o projections
    if s.moe is None:
        per_layer += 2.0 * T * s.hidden * 3 * s.ffn
    else:
        per_layer += 2.0 * T * s.hidden * (s.moe.num_experts + 3 * s.moe.top_k * s.moe.intermediate)
    keys = sum(range(past + 1, total + 1))
    attn = 2.0 * keys * s.num_q_heads * (s.k_dim + s.v_dim) * s.num_layers
    flops = per_layer * s.num_layers + attn + 2.0 * s.hidden * s.vocab               # last-token lm_head
    peak = float(measured_peaks().get("bf16_tflops", 1590.0))
    print(json.dumps({"measurement": "prefill_chunk_step", "model": shape.name, "chunk": T, "cached": past,
                      "ms_per_step": ms, "tokens_per_s": T / ms * 1e3, "tflop": flops / 1e12,
                      "tflops": flops / ms / 1e9, "frac_of_bf16_peak": flops / ms / 1e9 / peak,
                      "status": list(_lib.read_status())}))


def run_side_model(args, shape):
    """Side measurement (not the contract line): one decode step of another model shape (BASELINE
    configs 2, 3, 5: dense Qwen3 / Qwen2 shapes, the Moonlight MLA + MoE shape) on one GPU through the
    same stage runner and CUDA graph, against its own weights + KV HBM bound."""
    from vexact_b200 import _lib
    from vexact_b200.inferencer import StageRunner, StageWeights, StepInputs, allocate_kv_cache

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    S = args.batch
    weights = StageWeights.random_init(shape, 0, 1, device=device, seed=0)
    host, dev, nblocks = build_inputs(args, shape, seed=100, device=device)
    kc, vc = allocate_kv_cache(shape, 0, shape.num_layers, nblocks, args.page, device=device, fill_std=1.0, seed=0)
    runner = StageRunner(weights, kc, vc, 0, 1)
    inp = StepInputs(input_ids=dev["input_ids"], hidden_in=None, positions=dev["positions"],
                     slot_mapping=dev["slot_mapping"], query_start_loc=dev["query_start_loc"],
                     context_lens=dev["context_lens"], block_tables=dev["block_tables"], max_seqlen_q=1)
    _lib.reset_launch_count()
    runner.step(inp)
    torch.cuda.synchronize()
    launches = _lib.launch_count()
    graph, _ = runner.capture(inp)
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / args.steps
    kv_bytes = S * args.ctx * shape.num_kv_heads * (shape.k_dim + shape.v_dim) * 2 * shape.num_layers
    w_bytes = weights.num_bytes() - shape.vocab * shape.hidden * 2   # the embedding table is gathered, not streamed
    peak = float(measured_peaks().get("hbm_gbs", 6650.0))
    bound_ms = (kv_bytes + w_bytes) / peak / 1e6
    status = _lib.read_status()
    print(json.dumps({"measurement": "decode_step", "model": shape.name, "batch": S, "ctx": args.ctx,
                      "layers": shape.num_layers, "ms_per_step": ms, "tokens_per_s": S / ms * 1e3,
                      "weights_gb": w_bytes / 1e9, "kv_gb": kv_bytes / 1e9, "hbm_bound_ms": bound_ms,
                      "frac": bound_ms / ms, "launches_per_step": launches, "status": list(status)}))


def run_ragged_attention(args, shape):
    """Side measurement (not the contract line): one layer's decode attention over a ragged batch
    (context lengths uniform in [64, 2 * ctx]), with and without the longest-first sequence order."""
    import vexact_b200 as vb

    dev = torch.device("cuda", 0)
    hq, hkv, d, page, S = shape.num_q_heads, shape.num_kv_heads, shape.head_dim, args.page, args.batch
    g = torch.Generator().manual_seed(1)
    lens = torch.randint(64, 2 * args.ctx + 1, (S,), generator=g)
    pages = int((int(lens.max()) + page - 1) // page)
    gd = torch.Generator(device=dev).manual_seed(0)
    k_cache = torch.randn(S * pages, page, hkv, d, device=dev, generator=gd).bfloat16()
    v_cache = torch.randn(S * pages, page, hkv, d, device=dev, generator=gd).bfloat16()
    table = torch.randperm(S * pages, device=dev, generator=gd).view(S, pages).int()
    q = torch.randn(S, hq, d, device=dev, generator=gd).bfloat16()
    cu = torch.arange(S + 1, dtype=torch.int32, device=dev)
    used = lens.to(torch.int32).to(dev)
    order = torch.argsort(lens, descending=True, stable=True).to(torch.int32).to(dev)
    kv_bytes = int(lens.sum()) * hkv * 2 * d * 2
    res = {"measurement": "ragged_decode_attention", "sequences": S, "context": f"uniform 64..{2 * args.ctx}",
           "kv_bytes": kv_bytes}
    outs = []
    for name, so in (("unordered", None), ("longest_first", order)):
        call = lambda: vb.paged_attention(q, k_cache, v_cache, cu, used, table, d ** -0.5, 1, seq_order=so)
        for _ in range(max(args.warmup, 3)):
            outs.append(call())
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for _ in range(4):
                call()
        gr.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(max(args.steps, 1)):
            gr.replay()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / (4 * max(args.steps, 1))
        res[name] = {"ms": ms, "GBps": kv_bytes / ms / 1e6}
    res["same_bits"] = bool(torch.equal(outs[0], outs[-1]))
    print(json.dumps(res))


def zipf_router_bias(num_experts: int, seed: int, scale: float = 8.0) -> torch.Tensor:
    """Per-expert router-logit bias ~ Zipf(1.1) over a seeded random ranking of the experts (the skewed
    variant of the workload): rank r gets scale / r^1.1, so a few experts draw most of the tokens."""
    g = torch.Generator().manual_seed(seed)
    rank = torch.randperm(num_experts, generator=g).float() + 1.0
    return (scale / rank.pow(1.1)).to(torch.bfloat16)


def run_skew(args, shape):
    """Side measurement (not the contract line): the expert GEMMs of one MoE layer at batch `--batch`,
    under near-uniform routing (router std 0.02) and under the Zipf(1.1) router bias."""
    import vexact_b200 as vb
    from vexact_b200 import _lib
    from vexact_b200.fused_moe import FUSED_SWIGLU_MAX_ROWS_PER_EXPERT, _grouped_gemm, _permute

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    m, H, T = shape.moe, shape.hidden, args.batch
    E, k, I = m.num_experts, m.top_k, m.intermediate
    g = torch.Generator(device=dev).manual_seed(0)
    hidden = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    gate_up = (torch.randn(E, 2 * I, H, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    down = (torch.randn(E, H, I, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    router = (torch.randn(E, H, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    flush = torch.zeros(160 * 1024 * 1024, dtype=torch.float16, device=dev)     # 320 MB > L2
    peak = float(measured_peaks().get("hbm_gbs", 6650.0))

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            flush.add_(1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return sorted(ts)[len(ts) // 2] * 1e3      # us

    res = {"measurement": "moe_layer_skew", "model": shape.name, "tokens": T, "experts": E, "top_k": k}
    for name, bias in (("uniform", None), ("zipf_1.1", zipf_router_bias(E, seed=11).to(dev))):
        logits = vb.linear(hidden, router, bias)
        rw, sel = vb.route_softmax_topk(logits, k, True)
        counts = torch.bincount(sel.flatten(), minlength=E)
        plan = _permute(sel, rw, hidden, E)
        xp, rs = plan["x_perm"], plan["row_scale"]
        hit = int((counts > 0).sum())
        fused = T * k <= FUSED_SWIGLU_MAX_ROWS_PER_EXPERT * E
        fc1 = (lambda: _grouped_gemm(xp, gate_up, rs, plan, I, mode=1)) if fused else \
              (lambda: _grouped_gemm(xp, gate_up, None, plan, 2 * I, mode=0))
        hmid = _grouped_gemm(xp, gate_up, rs, plan, I, mode=1)
        e = {"rows_per_expert_max": int(counts.max()), "rows_per_expert_mean": float(counts.float().mean()),
             "experts_hit": hit, "token_tiles": int(plan["tile_count"].item()),
             "fc1_us": timed(fc1), "fc2_us": timed(lambda: _grouped_gemm(hmid, down, None, plan, H, mode=0)),
             "layer_us": timed(lambda: vb.fused_moe_forward(E, rw, sel, hidden, fc2_weight=down, fc1_1_2_weight=gate_up))}
        w1, w2 = hit * 2 * I * H * 2, hit * H * I * 2
        e["fc1_frac_of_hbm"] = (w1 + T * k * (H + I) * 2) / (e["fc1_us"] * 1e-6) / 1e9 / peak
        e["fc2_frac_of_hbm"] = (w2 + T * k * (H + I) * 2) / (e["fc2_us"] * 1e-6) / 1e9 / peak
        res[name] = e
    res["status"] = list(_lib.read_status())
    print(json.dumps(res))


def run_row_kernels(args, shape):
    """Side measurement (not the contract line): the HBM-bound row kernels at BASELINE config 1's shapes
    (hidden 2048, vocabulary 151936), each call on a fresh input (a ring of inputs larger than the L2), CUDA events."""
    from vexact_b200.batch_invariant_ops import batch_invariant_rms_norm, hf_rms_norm, log_softmax
    from vexact_b200.kv_cache_context import store_kvcache
    from vexact_b200.standalone_logprobs import logprobs_from_logits_flash_attn

    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    BF = torch.bfloat16
    out = {}

    def timed(name, calls, nbytes):
        for c in calls[:2]:
            c()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for c in calls:
            c()
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / len(calls)
        out[name] = {"us": round(us, 2), "bytes": nbytes, "GBps": round(nbytes / us / 1e3, 1)}

    rows, n, V = 16384, shape.hidden, shape.vocab
    w = torch.randn(n, device=dev, generator=g).to(BF)
    xs = [torch.randn(rows, n, device=dev, generator=g).to(BF) for _ in range(4)]        # 4 x 64 MB
    timed(f"rms_norm_{rows}x{n}", [lambda x=x: batch_invariant_rms_norm(x, w, 1e-6) for x in xs], rows * n * 4)
    timed(f"hf_rms_norm_{rows}x{n}", [lambda x=x: hf_rms_norm(x, w, 1e-6) for x in xs], rows * n * 4)
    M = 256
    ls = [torch.randn(M, V, device=dev, generator=g) * 2 for _ in range(3)]                # 3 x 156 MB fp32
    labels = torch.randint(0, V, (M,), device=dev, generator=g)
    timed(f"log_softmax_f32_{M}x{V}", [lambda x=x: log_softmax(x, -1) for x in ls], M * V * 8)
    timed(f"gather_logprob_f32_{M}x{V}", [lambda x=x: logprobs_from_logits_flash_attn(x, labels) for x in ls], M * V * 4)
    lb = [x.to(BF) for x in ls] + [x.to(BF) * 0.5 for x in ls]
    timed(f"gather_logprob_bf16_{M}x{V}", [lambda x=x: logprobs_from_logits_flash_attn(x, labels) for x in lb], M * V * 2)
    T, hkv, d, page = 16384, shape.num_kv_heads, shape.head_dim, args.page
    blocks = 4 * T // page
    kc = torch.zeros(blocks, page, hkv, d, device=dev, dtype=BF)
    vc = torch.zeros_like(kc)
    ks = [torch.randn(T, hkv, d, device=dev, generator=g).to(BF) for _ in range(4)]
    slots = [torch.randperm(T, device=dev, generator=g).int() + i * T for i in range(4)]
    timed(f"kv_store_{T}_tokens", [lambda k=k, sl=sl: store_kvcache(k, k, kc, vc, sl) for k, sl in zip(ks, slots)],
          T * hkv * d * 2 * 4)
    peak = float(measured_peaks().get("hbm_gbs", 6650.0))
    for v in out.values():
        v["frac_of_measured_hbm"] = round(v["GBps"] / peak, 3)
    print(json.dumps({"measurement": "row_kernels", "hbm_peak_GBps": peak, "kernels": out}))


def run_train_kernels(args, shape):
    """Side measurement (not the contract line): forward and forward + backward of the training-side calls, CUDA
    events: packed causal attention over 4 sequences of 2048 tokens, and one fused-MoE layer over 4096 tokens."""
    import vexact_b200 as vb

    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    BF = torch.bfloat16
    res = {}

    def timed(name, fn, reps=5):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        res[name] = round(a.elapsed_time(b) / reps, 3)

    hq, hkv, d = shape.num_q_heads, shape.num_kv_heads, shape.head_dim
    lens = [2048] * 4
    T = sum(lens)
    q = torch.randn(T, hq, d, device=dev, generator=g).to(BF).requires_grad_(True)
    k = torch.randn(T, hkv, d, device=dev, generator=g).to(BF).requires_grad_(True)
    v = torch.randn(T, hkv, d, device=dev, generator=g).to(BF).requires_grad_(True)
    dout = torch.randn(T, hq, d, device=dev, generator=g).to(BF)
    cu = torch.tensor([0, 2048, 4096, 6144, 8192], dtype=torch.int32, device=dev)

    def attn(backward):
        out, _ = vb.flash_attn_varlen_func(q, k, v, cu, cu, max_seqlen_q=2048, max_seqlen_k=2048, causal=True)
        if backward:
            out.backward(dout)

    with torch.no_grad():
        timed("attention_forward_ms", lambda: attn(False))
    timed("attention_forward_backward_ms", lambda: attn(True))
    if shape.moe is not None:
        E, kk, H, I = shape.moe.num_experts, shape.moe.top_k, shape.hidden, shape.moe.intermediate
        Tm = 4096
        x = torch.randn(Tm, H, device=dev, generator=g).to(BF).requires_grad_(True)
        w1 = (torch.randn(E, I, H, device=dev, generator=g) * 0.02).to(BF).requires_grad_(True)
        w2 = (torch.randn(E, I, H, device=dev, generator=g) * 0.02).to(BF).requires_grad_(True)
        w3 = (torch.randn(E, H, I, device=dev, generator=g) * 0.02).to(BF).requires_grad_(True)
        logits = torch.randn(Tm, E, device=dev, generator=g)
        rw, sel = vb.route_softmax_topk(logits, kk, True)
        rw = rw.requires_grad_(True)
        gy = torch.randn(Tm, H, device=dev, generator=g).to(BF)

        def moe(backward):
            out = vb.fused_moe_forward(E, rw, sel, x, w1, w2, w3)
            if backward:
                out.backward(gy)

        with torch.no_grad():
            timed("moe_forward_ms", lambda: moe(False))
        timed("moe_forward_backward_ms", lambda: moe(True))
        # the backward's GEMM forms on their own (vexact_b200.group_gemm), same shapes
        from vexact_b200 import group_gemm as gg
        with torch.no_grad():
            cu, _, si = vb.fused_moe.build_moe_indices(sel, E)
            ends, xs = cu[1:], gg.moe_scatter(x.detach(), si)
            h1 = gg.group_gemm_same_nk(xs, w1.detach(), ends, 0, transpose_b=True)
            gy8 = torch.randn(Tm * kk, H, device=dev, generator=g).to(BF)
            c1, c3 = torch.empty_like(w1), torch.empty_like(w3)
            timed("moe_plain_fc1_gemm_ms", lambda: gg.group_gemm_same_nk(xs, w1.detach(), ends, 0, transpose_b=True))
            timed("moe_dgrad_fc2_ms", lambda: gg.group_gemm_same_nk(gy8, w3.detach(), ends, 0, transpose_b=False))
            timed("moe_dgrad_fc1_ms", lambda: gg.group_gemm_same_nk(h1, w1.detach(), ends, 0, transpose_b=False))
            timed("moe_wgrad_fc2_ms", lambda: gg.group_gemm_same_mn(gy8, h1, c3, ends, 0, transpose_a=True,
                                                                    transpose_b=False))
            timed("moe_wgrad_fc1_ms", lambda: gg.group_gemm_same_mn(h1, xs, c1, ends, 0, transpose_a=True,
                                                                    transpose_b=False))
    print(json.dumps({"measurement": "train_kernels", "attention": {"tokens": T, "heads": [hq, hkv], "head_dim": d},
                      "ms": res}))


def run_prefill_attention(args, shape):
    """Side measurement (not the contract line): one sequence's causal prefill through paged attention."""
    import vexact_b200 as vb

    dev = torch.device("cuda", 0)
    hq, hkv, d, page = shape.num_q_heads, shape.num_kv_heads, shape.head_dim, args.page
    qlen = args.prefill_attention
    kvlen = max(qlen, args.ctx if args.ctx > qlen else qlen)
    pages = (kvlen + page - 1) // page
    g = torch.Generator(device=dev).manual_seed(0)
    k_cache = torch.randn(pages + 1, page, hkv, d, device=dev, generator=g).bfloat16()
    v_cache = torch.randn(pages + 1, page, hkv, d, device=dev, generator=g).bfloat16()
    table = torch.randperm(pages, device=dev, generator=g).view(1, pages).int()
    q = torch.randn(qlen, hq, d, device=dev, generator=g).bfloat16()
    cu = torch.tensor([0, qlen], dtype=torch.int32, device=dev)
    used = torch.tensor([kvlen], dtype=torch.int32, device=dev)
    call = lambda: vb.paged_attention(q, k_cache, v_cache, cu, used, table, d ** -0.5, qlen)
    for _ in range(max(args.warmup, 1)):
        call()
    torch.cuda.synchronize()
    # eager call: CUDA events around one call, i.e. with the host's launch path (three tensor-map encodes) inside
    eager = float("inf")
    for _ in range(max(args.steps, 1)):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        call()
        b.record()
        torch.cuda.synchronize()
        eager = min(eager, a.elapsed_time(b))
    # the kernel by itself: `reps` calls captured in one CUDA graph, replayed
    reps = 8
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps):
            call()
    graph.replay()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(max(args.steps, 1)):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b) / reps)
    keys = sum(range(kvlen - qlen + 1, kvlen + 1))          # causal (query, key) pairs
    flops = 2.0 * keys * hq * 2 * d                          # QK^T and PV
    print(json.dumps({"measurement": "prefill_attention", "queries": qlen, "context": kvlen, "heads": hq,
                      "kv_heads": hkv, "head_dim": d, "ms": best, "tflops": flops / best / 1e9,
                      "timing": "8 calls in a CUDA graph, per call", "eager_call_ms": eager,
                      "eager_call_tflops": flops / eager / 1e9}))


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    from vexact_b200.inferencer import PRESETS, ModelShape

    shape = PRESETS[args.model]
    if args.layers:
        shape = ModelShape(**{**shape.__dict__, "num_layers": args.layers})
    if args.impl == "reference":
        run_reference(args, shape, rank)
        return
    if args.skew:
        run_skew(args, shape)
        return
    if args.row_kernels:
        run_row_kernels(args, shape)
        return
    if args.train_kernels:
        run_train_kernels(args, shape)
        return
    if args.prefill_attention:
        run_prefill_attention(args, shape)
        return
    if args.ragged_attention:
        run_ragged_attention(args, shape)
        return
    if args.prefill_chunk:
        run_prefill_chunk(args, shape)
        return
    if args.model != "qwen3-30b-a3b-shape":
        run_side_model(args, shape)
        return

    import torch.distributed as dist

    import vexact_b200 as vb
    from vexact_b200 import _lib
    from vexact_b200.inferencer import StageRunner, StageWeights, StepInputs, allocate_kv_cache
    from vexact_b200.step_inputs import StepBuffers

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path for the product arm")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    _lib.load()
    pp = world
    if pp > 1:
        # a rank that dies must end the others' waits with an error, not leave the run hanging
        dist.init_process_group("nccl", device_id=device, timeout=__import__("datetime").timedelta(minutes=5))
    S, H = args.batch, shape.hidden
    watchdog = float(os.environ.get("B200_BENCH_WATCHDOG", "0") or 0)
    if watchdog > 0:      # debugging aid: every rank prints its Python stack if the run is still going by then
        import faulthandler

        faulthandler.dump_traceback_later(watchdog, exit=False, file=sys.stderr)

    def phase(name):
        if os.environ.get("B200_BENCH_TRACE"):
            print(f"[trace rank {rank}] {name} at {time.perf_counter() - t_start:.1f} s", file=sys.stderr, flush=True)

    t_start = time.perf_counter()

    weights = StageWeights.random_init(shape, rank, pp, device=device, seed=0)
    n_inflight = pp
    msg = None
    if pp > 1:
        from vexact_b200.config import PPInfo
        from vexact_b200.pp_messager import GenerationContext, InferencerOutput, PPMessager

        # one receive slot per batch in flight: batch b of every round lands at the same addresses, so
        # each later stage captures its graph directly on the received views (no copy on arrival)
        msg = PPMessager(PPInfo(pp, rank), None, device, recv_slots=n_inflight, send_slots=2,
                         group_timeout=__import__("datetime").timedelta(minutes=5))
    runners, graphs, outs, step_inputs, step_bufs, kv_blocks = [], [], [], [], [], []
    computed_host, tts_host = [args.ctx] * S, [1] * S    # per-request counters of a decode step
    first_ctx = [None] * n_inflight                       # stages > 0: the context a batch's graph was captured on
    for b in range(n_inflight):
        host, dev, nblocks = build_inputs(args, shape, seed=100 + b, device=device)
        kc, vc = allocate_kv_cache(shape, weights.start_layer, weights.end_layer, nblocks, args.page, device=device,
                                   fill_std=1.0, seed=b)
        runners.append(StageRunner(weights, kc, vc, rank, pp))
        runners[-1].fused_head = not args.unfused_head   # greedy token + logprob straight from the lm_head GEMM
        kv_blocks.append(nblocks)
        if rank == 0:
            # first stage: the step's buffers are built on the device from per-request counters
            # (b200_prepare_step); block tables and the previous step's tokens stay in HBM
            sb = StepBuffers(device, S, S, dev["block_tables"].shape[1], args.page)
            sb.request_blocks.copy_(dev["block_tables"])
            # decode input ids come from device memory (`last_tokens`); they keep their seeded random
            # values in every step so that the e2e leg routes tokens exactly as the device-timed leg does
            sb.last_tokens.copy_(dev["input_ids"])
            inp = sb.prepare([args.ctx] * S, [1] * S, None, S, S)
            for name, built in [("positions", inp.positions), ("slot_mapping", inp.slot_mapping),
                                ("query_start_loc", inp.query_start_loc), ("context_lens", inp.context_lens),
                                ("block_tables", inp.block_tables), ("input_ids", inp.input_ids)]:
                if not torch.equal(built, dev[name]):
                    raise SystemExit(f"device-built {name} differs from the host-built one")
            step_bufs.append(sb)
            step_inputs.append(inp)
    if pp > 1:
        W = (args.ctx + args.page - 1) // args.page
        msg.reserve(H, S, S, W, 0)
    torch.cuda.synchronize()

    def ctx_of(inp, hidden):
        """The context a stage hands on: its output hidden states plus the step's metadata."""
        return GenerationContext(batch_input_ids=None, intermediate_tensors=hidden[None],
                                 query_start_loc=inp.query_start_loc, batch_position_ids=inp.positions[None],
                                 block_tables=inp.block_tables, context_lens=inp.context_lens,
                                 slot_mapping=inp.slot_mapping, max_seqlen_q=1)

    no_delta = tuple(torch.empty(0, dtype=torch.int32, device=device) for _ in range(3))

    def hand_on(b, inp, out, first):
        """Stage output -> next stage (context) or, on the last stage, tokens + logprobs -> first stage."""
        if rank < pp - 1:
            # the block table travels whole once per batch slot, then as deltas (none in a decode step
            # that stays inside its last page)
            msg.send_gen_ctx(ctx_of(inp, out), slot=b, block_delta=None if first else no_delta)
        else:
            msg.send_infer_out(InferencerOutput(token_ids=out[0], logits=torch.empty(0, device=device),
                                                logprobs=out[1]))

    def inputs_from(ctx):
        return StepInputs(input_ids=None, hidden_in=ctx.intermediate_tensors[0], positions=ctx.batch_position_ids[0],
                          slot_mapping=ctx.slot_mapping, query_start_loc=ctx.query_start_loc,
                          context_lens=ctx.context_lens, block_tables=ctx.block_tables, max_seqlen_q=1)

    # ---- set-up round: one eager step per batch flows down the pipeline; every stage counts its launches
    # and captures its graph on the buffers the step arrived in
    launches_per_step = 0
    for b in range(n_inflight):
        if rank > 0:
            first_ctx[b] = msg.recv_gen_ctx()
            step_inputs.append(inputs_from(first_ctx[b]))
        _lib.reset_launch_count()
        out = runners[b].step(step_inputs[b])
        torch.cuda.synchronize()
        launches_per_step = _lib.launch_count()
        if args.no_graph:
            graphs.append(None)
            outs.append(None)
        else:
            gr, out = runners[b].capture(step_inputs[b])
            graphs.append(gr)
            outs.append(out)
            gr.replay()
        if pp > 1:
            hand_on(b, step_inputs[b], out, first=True)
    phase("set-up round done")
    pending = [pp > 1 and rank == 0] * n_inflight   # rank 0: a token message of the batch's previous step is owed
    status = _lib.read_status()
    if status[0] != 0:
        raise SystemExit(f"device status word reports {status}")

    def run_stage(b):
        if graphs[b] is not None:
            graphs[b].replay()
            return outs[b]
        return runners[b].step(step_inputs[b])

    # e2e results land in two pinned buffers in turn: the host reads step N's tokens while step N + 1
    # runs (its inputs need only the requests' lengths; the token ids themselves stay on the device)
    tok_host = [torch.empty(S, dtype=torch.int64).pin_memory() for _ in range(2)]
    lp_host = [torch.empty(S, dtype=torch.float32).pin_memory() for _ in range(2)]
    e2e_done = [torch.cuda.Event(), torch.cuda.Event()]
    e2e_count = [0]
    trace = [] if os.environ.get("B200_BENCH_TRACE") else None

    def global_step(e2e=False):
        """Advance every in-flight batch by one token through this rank's stage."""
        for b in range(n_inflight):
            if rank == 0:
                if pending[b]:                  # tokens + logprobs of this batch's previous step
                    msg.recv_infer_out()
                    pending[b] = False
                if e2e:                         # counters up, one kernel builds the step's buffers
                    step_bufs[b].prepare(computed_host, tts_host, None, S, S)
            else:
                ctx = msg.recv_gen_ctx()        # lands where this batch's graph reads its inputs
                if ctx.intermediate_tensors.data_ptr() != first_ctx[b].intermediate_tensors.data_ptr():
                    raise SystemExit("a batch's context arrived at another address than its graph was captured on")
            if trace is not None:
                trace.append((torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)))
                trace[-1][0].record()
            out = run_stage(b)
            if trace is not None:
                trace[-1][1].record()
            if pp > 1:
                hand_on(b, step_inputs[b], out, first=False)
            if rank == pp - 1 and e2e:
                tok_host[e2e_count[0] & 1].copy_(out[0], non_blocking=True)
                lp_host[e2e_count[0] & 1].copy_(out[1], non_blocking=True)
            if pp > 1 and rank == 0:
                pending[b] = True               # one token message is now owed to this batch
        if e2e:
            e2e_done[e2e_count[0] & 1].record()
            if e2e_count[0] > 0:
                e2e_done[(e2e_count[0] - 1) & 1].synchronize()   # the previous step's results are on the host
            e2e_count[0] += 1

    def drain():
        for b in range(n_inflight):
            if pending[b]:
                msg.recv_infer_out()
                pending[b] = False
        if msg is not None:
            msg.flush()

    def sync_all():
        drain()
        torch.cuda.synchronize()
        if pp > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if not args.quick:
        sampler.start()
        sampler.wait_first_sample()
    sync_all()
    phase("pipeline drained after set-up")
    for _ in range(max(args.warmup, 3) if not args.quick else args.warmup):
        global_step()
    if pp == 1:
        sync_all()
    phase("warm-up done")

    # ---- device-timed run (inputs resident in HBM; weights + KV >> L2, so every step is cold).
    # With pipeline stages the warm-up steps run straight into the timed ones (no drain in between), so
    # the pipeline is full when a rank's first timed stage starts; each rank times its own K steps.
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    first_sample = sampler.mark()
    ev0.record()
    for _ in range(args.steps):
        global_step()
    ev1.record()
    sync_all()
    phase("device-timed steps done")
    dev_ms = ev0.elapsed_time(ev1)
    if trace is not None:
        tail = trace[-args.steps * n_inflight:]
        st = [a.elapsed_time(b) for a, b in tail]
        gaps = [tail[i][1].elapsed_time(tail[i + 1][0]) for i in range(len(tail) - 1)]
        print(f"[trace rank {rank}] stage ms mean {sum(st) / len(st):.3f} max {max(st):.3f}; "
              f"gap ms mean {sum(gaps) / max(len(gaps), 1):.3f} max {max(gaps) if gaps else 0:.3f}; "
              f"step {dev_ms / args.steps:.3f}", file=sys.stderr, flush=True)
        trace.clear()
    if args.quick:
        if rank == 0:
            print(json.dumps({"quick": True, "ms_per_step": dev_ms / args.steps,
                              "value": S * n_inflight * args.steps / (dev_ms * 1e-3)}), flush=True)
        if pp > 1:
            dist.destroy_process_group()
        return

    # ---- end-to-end run: pinned host inputs in, tokens + logprobs out, every step
    h2d = step_bufs[0].h2d_bytes_last_step if rank == 0 else 0   # per-request counters (3 x int32 per sequence)
    d2h = (tok_host[0].numel() * 8 + lp_host[0].numel() * 4) if rank == pp - 1 else 0

    def e2e_step():
        global_step(e2e=True)

    for _ in range(2):
        e2e_step()
    if pp == 1:
        sync_all()
    else:
        torch.cuda.synchronize()   # this rank's own queue only: the pipeline stays full
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    if pp == 1:
        sync_all()
    else:
        torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    sync_all()
    if trace is not None:
        tail = trace[-args.steps * n_inflight:]
        st = [a.elapsed_time(b) for a, b in tail]
        gaps = [tail[i][1].elapsed_time(tail[i + 1][0]) for i in range(len(tail) - 1)]
        print(f"[trace rank {rank}, e2e] stage ms mean {sum(st) / len(st):.3f} max {max(st):.3f}; "
              f"gap ms mean {sum(gaps) / max(len(gaps), 1):.3f} max {max(gaps) if gaps else 0:.3f}",
              file=sys.stderr, flush=True)
        trace = None
    clocks = sampler.stop(first_sample)

    # ---- dominant kernel alone (paged decode attention over every local layer's cache)
    att = {}
    r0 = runners[0]
    if rank > 0:   # later stages: their metadata arrived over the wire
        step_inputs[0] = inputs_from(first_ctx[0])
    q = torch.randn(S, shape.num_q_heads, shape.head_dim, device=device).to(torch.bfloat16)
    layers = list(range(weights.start_layer, weights.end_layer))
    reps = max(2, min(args.steps, 5))

    def attn_all():
        for li in layers:
            vb.paged_attention(q, r0.key_cache[li], r0.value_cache[li], step_inputs[0].query_start_loc,
                               step_inputs[0].context_lens, step_inputs[0].block_tables, shape.head_dim ** -0.5, 1)

    attn_all()
    torch.cuda.synchronize()
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0.record()
    for _ in range(reps):
        attn_all()
    a1.record()
    torch.cuda.synchronize()
    att_ms = a0.elapsed_time(a1) / (reps * len(layers))
    kv_bytes = S * args.ctx * shape.num_kv_heads * 2 * shape.head_dim * 2
    att_bytes = kv_bytes + 2 * S * shape.num_q_heads * shape.head_dim * 2 + 4 * S * (step_inputs[0].block_tables.shape[1] + 2)
    peaks = measured_peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = att_bytes / (att_ms * 1e-3) / 1e9
    kernel_name = "paged_attn_tc_kernel<128,128,16,3,3>"
    ncu_traffic = recorded_traffic(kernel_name, S, args.ctx, args.page)
    att = {"bound": "hbm", "kernel": kernel_name, "achieved": achieved, "peak": peak,
           "peak_source": "MEASURED_PEAKS.json" if peaks else "fallback 6650 GB/s", "unit": "GB/s",
           "frac": achieved / peak, "traffic": ncu_traffic, "algorithmic_bytes_per_launch": att_bytes,
           "ms_per_launch": att_ms}

    # ---- gather timing across ranks (max), emit
    t = torch.tensor([dev_ms, e2e_s * 1e3, float(h2d), float(d2h)], device=device, dtype=torch.float64)
    if pp > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, h2d, d2h = t.tolist()
    h2d, d2h = int(h2d), int(d2h)
    tokens_per_step = S * n_inflight
    value = tokens_per_step * args.steps / (dev_ms * 1e-3)
    e2e_value = tokens_per_step * args.steps / (e2e_ms * 1e-3)
    step_bytes = weights.num_bytes() + len(layers) * kv_bytes
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(args, shape), "pipeline_stages": pp, "batches_in_flight": n_inflight,
                   "l2": "inputs (weights + KV, >100 GB per GPU) far exceed L2; no flush needed",
                   "cuda_graph": not args.no_graph,
                   "handoff": ("PPMessager.send_gen_ctx / recv_gen_ctx / send_infer_out: hidden states + step metadata "
                               "(positions, slot mapping, query_start_loc, context lengths, block-table deltas) every step; "
                               "pipeline kept full across the timed region, each rank times its own steps") if pp > 1 else "none",
                   "e2e": "per step: H2D of per-request counters, device-built inputs, graph replay, D2H of tokens + logprobs; the host reads step N's results while step N+1 runs"},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d * n_inflight,
                "d2h_bytes_per_step": d2h * n_inflight, "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": launches_per_step * n_inflight * args.steps,
        "roofline": att,
        "step_roofline": {"bytes_per_stage_step": step_bytes, "hbm_bound_ms": step_bytes / (peak * 1e9) * 1e3,
                          "frac": (step_bytes / (peak * 1e9) * 1e3) / (dev_ms / args.steps / n_inflight)},
    }
    if rank == 0 and pp == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        seqs = min(S, 128)
        sam = CpuSample(args, shape, seqs, threads)
        sam.run()
        secs = min(sam.run() for _ in range(2))
        v = seqs / secs
        line["cpu_baseline"] = {
            "value": v, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": (f"1 of {shape.num_layers} decoder layers (time x {shape.num_layers}) + head, {seqs} of "
                       f"{S} sequences at ctx {args.ctx}, torch CPU ops; extrapolated step {secs:.2f} s"),
        }
    if rank == 0:
        print(json.dumps(line), flush=True)
    if pp > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
