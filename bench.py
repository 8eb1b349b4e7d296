"""bench.py: tokens/s of a Llama-7B-shaped prefill on N B200s (one process a GPU).

A step is one call of the model's `loss` entry (prefill + next-token loss) on one
batch of synthetic token ids, through the host program of libpresk_cuda.so.

  value   tokens/s over all ranks with the ids already on the device, timed with
          CUDA events on the executor's stream, the maximum over ranks
  e2e     the same through the C ABI with pinned HOST buffers: the host-to-device
          copy of the ids and labels, the gather of the loss over the ranks (one
          all-reduce) and its device-to-host read are inside the timed region of
          every step
  roofline  the tensor-core contraction kernel: its floating-point operations over its
          own time (events around every launch of the timed steps), against the
          measured cuBLAS bf16 rate of MEASURED_PEAKS.json
  parity  a pre-flight outside the timed region: one layer of the workload's width
          over the CUDA executor (the benchmark's realization) and over the CPU oracle
          (sequential order), logits and loss compared; rank 0 only
  cpu_baseline  the CPU restatement of the same launches (oracle/, OpenMP over the
          host's cores) on a bounded sample, rank 0 and N = 1 only

`--impl reference` times that CPU path alone, on the same metric, with one layer at
the workload's own sequence length among its samples.

`--workload` also takes the smaller configurations (the MLP classifier, the small
GPT, the contraction-plus-LayerNorm sweep); each prints the same JSON shape.

The batch axis is sharded over the ranks with no collective on the data path; the
per-rank losses are combined with one all-reduce a step (`--comm psk`: the library's
own psk_comm_* over NCCL on the executor's stream; `--comm torch`: torch.distributed).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # the Llama-7B-shaped prefill: 32 layers, d 4096, 32 heads of 128, SwiGLU 11008, vocab 32000, seq 2048, batch 8 a GPU
    "llama7b_prefill_b8_t2048": dict(consts=dict(V=32000, D=4096, H=32, G=32, FF=11008, L=32), B=8, T=2048),
    # its int8 variant: the same architecture, projection and FFN weights int8 with one f32 scale a
    # channel, bf16 activations, seq 1024, batch 16 a GPU
    "llama7b_int8_prefill_b16_t1024": dict(consts=dict(V=32000, D=4096, H=32, G=32, FF=11008, L=32), B=16, T=1024, int8=True),
    "llama7b_w8a8_prefill_b16_t1024": dict(consts=dict(V=32000, D=4096, H=32, G=32, FF=11008, L=32), B=16, T=1024, int8="w8a8"),
    "llama7b_w8a8_prefill_b8_t2048": dict(consts=dict(V=32000, D=4096, H=32, G=32, FF=11008, L=32), B=8, T=2048, int8="w8a8"),
    # and with those weights stored e4m3fn (a `params` entry; the reference has no scale for such weights, so N(0, 0.02)
    # keeps about three significant bits): the same launches, the weights widened exactly
    "llama7b_e4m3w_prefill_b16_t1024": dict(consts=dict(V=32000, D=4096, H=32, G=32, FF=11008, L=32), B=16, T=1024, int8="e4m3fn"),
    # a small shape of the same program, for trying the script out
    "llama_small": dict(consts=dict(V=4096, D=1024, H=8, G=8, FF=2816, L=4), B=4, T=512),
    # generation: one new token a sequence against a cache of 1024 positions' keys and values (the reference's serve loop
    # recomputes the window for every token, presk-serve/src/lib.rs:241; this keeps them), batch 16 a GPU
    "llama7b_decode_b16_ctx1024": dict(kind="decode", consts=dict(V=32000, D=4096, H=32, G=32, FF=11008, L=32), B=16, T=1024),
    "llama_small_decode": dict(kind="decode", consts=dict(V=4096, D=1024, H=8, G=8, FF=2816, L=4), B=4, T=256),
    # the 2-layer ReLU MLP classifier: Linear{784,256}, ReLU, Linear{256,10}, cross-entropy; batch 4096; all f32 (sequential order: the reference's bits)
    "mlp_b4096": dict(kind="mlp", B=4096),
    # the small GPT decoder: 4 layers, d 128, 4 heads, context 64, vocabulary 65, batch 256; a mixed bf16/f32 assignment
    "gpt_l4_d128_b256_t64": dict(kind="gpt", consts=dict(V=65, D=128, H=4, L=4), B=256, T=64),
}
# x[N, N]·w[N, N] then a row LayerNorm, every site stored f16 or e8m15, computed in f32
for _n in (1024, 4096, 8192):
    for _dt in ("f16", "e8m15"):
        WORKLOADS[f"contract_ln_{_n}_{_dt}"] = dict(kind="contract_ln", N=_n, dtype=_dt)


QUANTISED = ("blocks.attn.wq", "blocks.attn.wk", "blocks.attn.wv", "blocks.attn.wo", "blocks.ff.gate.w", "blocks.ff.up.w", "blocks.ff.down.w")


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel's heaviest frequent shape, from the
# ncu capture summarised in profiles/k_gemm_tc_ffn_16384x11008x4096.md (bytes a launch; algorithmic bytes: 585 MB)
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the step's dominant kernel under ncu (profiles/)
GEMM_TRAFFIC = {"llama7b_prefill_b8_t2048": 791255040 + 335562752, "llama7b_w8a8_prefill_b8_t2048": 188421120 + 325028096, "llama7b_w8a8_prefill_b16_t1024": 188421120 + 325028096}
GEMM_TRAFFIC_OF = "dot [16384, 4096] x [4096, 11008] (gate/up projections: 64 of a step's 225 contractions), one launch under ncu: k_gemm_tc<256, false, 2, false, 1> for bf16, k_gemm_i8<1> for the W8A8 workloads"


def realization(paths, int8=False, attention="unfused", launches="reference"):
    """A solved-style mixed bf16/f32 assignment: bf16 storage, f32 where a sum's result is reused
    widely (the norms' mean and root, the logits and the loss); with `int8`, the projection and
    FFN weights as integers with one scale a channel (`quant`, over the contracted axis); with `int8` the
    string "e4m3fn", those weights stored e4m3fn instead (`params`)."""
    rz = {
        "default": "bf16",
        "order": {"kind": "device", "attention": attention, "launches": launches},
        "params": {p: ("e4m3fn" if int8 == "e4m3fn" and p in QUANTISED else "bf16") for p in paths if not (int8 is True and p in QUANTISED)},
        "storage": {"RMSNorm.apply/%3": "f32", "RMSNorm.apply/%7": "f32", "Llama.apply/%11": "f32", "loss/%5": "f32", "loss/%6": "f32"},
    }
    if int8 is True:
        rz["quant"] = {p: {"bits": 8, "over": -2} for p in QUANTISED}
    return rz


# W8A8: the projections' inputs (the norm's result, silu(gate)·up) stored as i8 codes with static scales, every
# projection's weights and the head's as int8, those contractions' products and sums counted in i32: the integer-sum
# kernel on tcgen05's 8-bit kind. Under `attention: online` with merged launches the attention's result is a scaled
# site too (the one-pass kernel writes the codes) and the out-projection counts in i32 like the other six; under the
# other attention orders it stays bf16 and the out-projection widens its int8 weights.
W8A8_SCALED = ("RMSNorm.apply/%10", "SwiGLU.apply/%7")
W8A8_INT_SUMS = ("Attention.apply/%7", "Attention.apply/%11", "Attention.apply/%14", "Dense.apply/%3", "Llama.apply/%11")
W8A8_ATTN_OUT_SITE, W8A8_ATTN_OUT_SUMS = "Attention.apply/%22", "Attention.apply/%26"


def w8a8_attention_in_codes(attention, launches):
    return attention == "online" and launches == "merged"


def w8a8_realization(paths, attention, launches, scales):
    quantised = QUANTISED + ("head",)
    codes = w8a8_attention_in_codes(attention, launches)
    scaled = W8A8_SCALED + ((W8A8_ATTN_OUT_SITE,) if codes else ())
    sums = W8A8_INT_SUMS + ((W8A8_ATTN_OUT_SUMS,) if codes else ())
    rz = realization(paths, False, attention, launches)
    rz["params"] = {p: "bf16" for p in paths if p not in quantised}
    rz["quant"] = {p: {"bits": 8, "over": -2} for p in quantised}
    rz["scaled"] = {site: {"int": "i8/sat", "scale": float(np.float32(scales[site])), "zero": 0} for site in scaled}
    rz["product"] = {site: "i32" for site in sums}
    rz["accum"] = {site: "i32" for site in sums}
    return rz


def param_shapes(c):
    V, D, FF, L, H = c["V"], c["D"], c["FF"], c["L"], c["H"]
    G = c.get("G", H)
    HD = D // H
    return {
        "tok": ((V, D), 0.02), "head": ((D, V), 0.02), "norm.γ": ((D,), -1.0),
        "blocks.n1.γ": ((L, D), -1.0), "blocks.n2.γ": ((L, D), -1.0),
        "blocks.attn.wq": ((L, D, D), 0.02), "blocks.attn.wk": ((L, D, G * HD), 0.02), "blocks.attn.wv": ((L, D, G * HD), 0.02), "blocks.attn.wo": ((L, D, D), 0.02),
        "blocks.ff.gate.w": ((L, D, FF), 0.02), "blocks.ff.up.w": ((L, D, FF), 0.02), "blocks.ff.down.w": ((L, FF, D), 0.02),
    }


def flops_per_token(c, T):
    D, FF, L, V = c["D"], c["FF"], c["L"], c["V"]
    return L * (8 * D * D + 6 * D * FF + 4 * T * D) + 2 * D * V


class ClockSampler:
    """nvidia-smi sampled every 200 ms while the timed region runs."""

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q, "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        reasons = set()
        for r in self.rows:
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def time_call(fn, warmup=1, reps=3):
    """The reference's timing protocol (presk-driver/src/bench.rs:28-48): untimed warm-up calls, then the
    median of `reps` timed ones. Returns (median seconds, every timing)."""
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    return statistics.median(ts), ts


def cpu_prefill_tokens_per_s(consts, T, B, threads, int8=False, direct=False, direct_budget_s=240.0):
    """The CPU restatement of the prefill on a bounded sample of the workload, every timing a median of three
    after a warm-up call:

      * one and three layers of the full width at B = 1, T = 128 (a median of five each: the per-layer time is
        half their difference, which is multiplied by the depth afterwards, so its noise matters most): the
        per-layer time and the rest (embedding, final norm, head, loss), both proportional to the number of tokens;
      * the attention function at the workload's own T and at 128 on 16 heads of 128 (32 on a host of more than
        16 threads): the part of a layer that grows with T squared, per head (every head does the same work on
        its own [T, 128] operands);
      * with `direct` (the reference arm): one layer of the full width at B = 1 and the workload's T, the whole
        thing, so that attention's share at that length is measured and not modelled.

    tokens/s of the whole depth = B·T / (B · (rest + L · layer)), every term scaled to T tokens."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import headline
    import oracle_lib
    from presk_b200 import Host

    # all the host's cores, also under torchrun (which sets OMP_NUM_THREADS=1 for its workers);
    # set before the OpenMP runtime of the oracle's library is loaded
    os.environ["OMP_NUM_THREADS"] = str(threads)
    orc = oracle_lib.load()
    rng = np.random.default_rng(0)
    Ts = min(T, 128)
    # (the W8A8 workload's CPU leg runs the W8A16 realization: the same int8 weights against bf16 activations)
    weights = "int8" if int8 in (True, "w8a8") else ("e4m3fn" if int8 == "e4m3fn" else "bf16")
    fmt = lambda ts: "[" + ", ".join(f"{t:.2f}" for t in ts) + "]"

    LN = 3
    c2 = dict(consts, L=LN)
    p2 = headline.llama_params_f32(c2, seed=0)
    ids = rng.integers(0, consts["V"], size=(1, Ts), dtype=np.int64)
    y = rng.integers(0, consts["V"], size=(1, Ts), dtype=np.int64)
    med, raw = {}, {}
    hosts = {}
    for L in (1, LN):
        c = dict(consts, L=L)
        p = {k: (np.ascontiguousarray(v[:L]) if k.startswith("blocks.") else v) for k, v in p2.items()}
        h = headline.give(Host(orc.vtable(), headline.realization(p, headline.ORACLE_ORDER, weights)).prepare("llama", **c), p)
        med[L], raw[L] = time_call(lambda: h.call("loss", [ids, y], ()), reps=5)
        if L == 1 and direct:
            hosts[1] = h
        else:
            h.close()
    # the part of a layer that grows with T squared, per head: a few heads of 128 at T and at 128
    # (as many heads as keep every thread busy: the oracle divides the (batch, head) loop over the threads)
    hs = min(consts["H"], 32 if threads > 16 else 16)
    ca = dict(V=64, D=128 * hs, H=hs, G=hs, FF=256, L=1)
    pa = headline.llama_params_f32(ca, seed=1)
    ha = headline.give(Host(orc.vtable(), headline.realization(pa, headline.ORACLE_ORDER)).prepare("llama", **ca), pa)
    xa = {t: rng.standard_normal((1, t, ca["D"])).astype(np.float32) for t in {Ts, T}}
    att = {t: time_call(lambda t=t: ha.call("attention", [xa[t]], (1, t, ca["D"]))) for t in sorted(xa)}
    ha.close()
    if T > Ts:
        quad_head = max((att[T][0] - att[Ts][0] * (T / Ts)) / ((T * T - T * Ts) * ca["H"]), 0.0)  # seconds a head a (token pair)
    else:
        quad_head = 0.0
    heads = consts["H"]
    layer_s = max((med[LN] - med[1]) / (LN - 1), 1e-9)
    rest_s = max(med[1] - layer_s, 0.0)
    lin_layer_s = max(layer_s - heads * quad_head * Ts * Ts, 0.0)
    up = T / Ts
    layer_T_model = lin_layer_s * up + heads * quad_head * T * T
    rest_T = rest_s * up
    sample = (f"oracle (C restatement, OpenMP, {threads} threads), warm-up 1 + median of 3 each (of 5 for the layers); B=1, T={Ts}: L=1 {fmt(raw[1])} s, L={LN} {fmt(raw[LN])} s"
              f" => layer {layer_s:.2f} s, rest {rest_s:.2f} s; attention function on {hs} heads of 128: T={Ts} {fmt(att[Ts][1])} s"
              + (f", T={T} {fmt(att[T][1])} s => {heads * quad_head * T * T:.1f} s a layer of {heads} heads at T={T}" if T > Ts else "")
              + f"; modelled layer at T={T}: {layer_T_model:.1f} s")
    layer_T = layer_T_model
    if direct:
        # one whole layer of the full width at the workload's own sequence length
        idsT = rng.integers(0, consts["V"], size=(1, T), dtype=np.int64)
        yT = rng.integers(0, consts["V"], size=(1, T), dtype=np.int64)
        h1 = hosts[1]
        t_start = time.perf_counter()
        t0 = time.perf_counter()
        h1.call("loss", [idsT, yT], ())
        warm = time.perf_counter() - t0
        ts = []
        while len(ts) < 3 and (time.perf_counter() - t_start) + warm <= direct_budget_s:
            t0 = time.perf_counter()
            h1.call("loss", [idsT, yT], ())
            ts.append(time.perf_counter() - t0)
        h1.close()
        whole = statistics.median(ts) if ts else warm
        layer_T = max(whole - rest_T, 1e-9)
        sample += (f"; measured whole L=1, B=1, T={T}: warm-up {warm:.1f} s, timed {fmt(ts)} s"
                   + ("" if ts else " (no timed call fitted the time limit: the warm-up call is used)")
                   + f" => layer {layer_T:.1f} s (used)")
    full = rest_T + consts["L"] * layer_T
    sample += f"; extrapolated to L={consts['L']}: {full:.0f} s a sequence"
    return T / full, sample


def microbench(args):
    """One kernel alone on synthetic operands, for tuning and for profiler captures:
    `--micro gemm --shape M,N,K[,batch[,b_n_major]]`, `--micro softmax --shape rows,n`,
    `--micro ew --shape rows,cols`, `--micro attn --shape batch,heads,seq` (hd = 128, causal), `--micro norm --shape rows,cols`.
    Prints one JSON line (not the benchmark's)."""
    import torch
    from presk_b200 import Executor, abi, launch_desc

    ex = Executor(0)
    stream = torch.cuda.ExternalStream(ex.stream())
    dims = [int(x) for x in args.shape.split(",")]
    rng = np.random.default_rng(0)

    def bf16(shape):
        a = rng.standard_normal(shape).astype(np.float32)
        return (a.view(np.uint32) >> 16).astype(np.uint16)

    def timed(fn, reps):
        for _ in range(3):
            fn()
        ex.sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            fn()
        e1.record(stream)
        ex.sync()
        return e0.elapsed_time(e1) / reps

    if args.micro == "train":
        # one training step (loss_grad + adamw.step) of a Llama-shaped model under the device order, bf16 storage:
        # --shape V,D,H,FF,L,B,T. Not the benchmark's metric: the reverse pass is not tuned.
        from presk_b200 import Host
        V, D, H, FF, L, B, T = dims[:7]
        consts = dict(V=V, D=D, H=H, G=H, FF=FF, L=L)
        shapes = param_shapes(consts)
        rz = realization(shapes, False, "unfused", "reference")
        rz["functions"] = {"adamw.step": "f32", "adamw.lr": "f32"}  # moments and the schedule in f32; parameters stay bf16
        host = Host(ex, rz).prepare("llama", **consts).adamw(lr=1e-4, weight_decay=0.1, grad_clip=1.0)
        for i, (path, (shape, std)) in enumerate(shapes.items()):
            if std < 0:
                host.set_param(path, np.ones(shape, np.float32))
            else:
                host.init_param(path, 1000 + i, std, shape)
        ids = rng.integers(0, V, size=(B, T), dtype=np.int64)
        y = rng.integers(0, V, size=(B, T), dtype=np.int64)
        step = [0]
        dev_in = [(ex.upload(ids), abi.I64, (B, T)), (ex.upload(y), abi.I64, (B, T))]

        def one():
            # inputs resident and the gradient left on the executor, as a training loop has them (the host-buffer
            # call would bring the first leaf, half a gigabyte, back to the host every step)
            step[0] += 1
            host.call_device("loss_grad", dev_in)
            host.adamw_step(step[0], 1000)

        for _ in range(2):
            one()
        ex.sync()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            one()
        ex.sync()
        ms = (time.perf_counter() - t0) * 1e3 / args.steps
        flops = 3.0 * flops_per_token(consts, T) * B * T
        ex.set_profiling(True)
        one()
        agg = {}
        singles = []
        for kern, name, kms, _, nbytes in ex.profile():
            a = agg.setdefault(kern + " | " + name, [0, 0.0])
            a[0] += 1
            a[1] += kms
            singles.append((kms, kern + " | " + name, nbytes))
        ex.set_profiling(False)
        if os.environ.get("PSK_BENCH_SINGLES"):
            # the launches furthest below the memory's rate, one by one: where a generic kernel ran
            worst = sorted(singles, key=lambda r: -r[0])[:int(os.environ["PSK_BENCH_SINGLES"])]
            print(json.dumps({"slowest_launches [ms, name, MB, GB/s]": [[round(m_, 3), n_, round(b_ / 1e6, 1), round(b_ / 1e6 / m_, 1) if m_ else None] for m_, n_, b_ in worst]}))
        top = sorted(agg.items(), key=lambda kv: -kv[1][1])[:14]
        print(json.dumps({"top_launches_ms": {k: [v[0], round(v[1], 3)] for k, v in top}, "profiled_total_ms": round(sum(v[1] for v in agg.values()), 2)}))
        print(json.dumps({"micro": "train", "shape": dims, "ms_per_step": ms, "tokens/s": B * T / ms * 1e3, "model TFLOP/s (3x forward)": flops / ms / 1e9, "loss": float(host.call("loss", [ids, y], ()))}))
        return
    if args.micro == "gemm":
        m, n, k = dims[:3]
        batch = dims[3] if len(dims) > 3 else 1
        bnm = dims[4] if len(dims) > 4 else 0
        a, b = ex.upload(bf16((batch, m, k))), ex.upload(bf16((batch, n, k)))
        c = ex.alloc(batch * m * n * 2)
        g = abi.Gemm()
        g.in_dtype, g.out_dtype, g.b_n_major = abi.BF16, abi.BF16, bnm
        g.m, g.n, g.k, g.batch, g.batch_lo = m, n, k, batch, batch
        g.a_row, g.a_lo, g.a_hi = k, m * k, m * k * batch
        g.b_row, g.b_lo, g.b_hi = (n if bnm else k), n * k, n * k * batch
        g.c_row_lo_count, g.c_row_lo, g.c_col_lo_count = m, n, n
        g.c_lo, g.c_hi = m * n, m * n * batch
        ms = timed(lambda: ex.gemm(g, a, b, c), args.steps)
        fl = 2.0 * m * n * k * batch
        print(json.dumps({"micro": "gemm", "shape": dims, "ms": ms, "TFLOP/s": fl / ms / 1e9, "GB/s": (batch * (m * k + n * k + m * n) * 2) / ms / 1e6}))
    elif args.micro == "gemm_i8":
        # the integer-sum contraction: i8 activation codes [m, k] (one scale) times int8 weights [k, n] (a scale a column), bf16 result
        m, n, k = dims[:3]
        a = ex.upload(rng.integers(-128, 128, size=(m, k), dtype=np.int8))
        b = ex.upload(rng.integers(-127, 128, size=(k, n), dtype=np.int8))
        sw = ex.upload((rng.uniform(1.0, 2.0, size=n) * 2.0 ** -8).astype(np.float32))
        c = ex.alloc(m * n * 2)
        add = len(dims) > 4 and dims[4] == 1  # 5th number 1: a bf16 residual [m, n] added in the kernel's epilogue (PSK_OP_CONTRACT_ADD)
        l = launch_desc(abi.OP_CONTRACT_ADD if add else abi.OP_CONTRACT, abi.BF16, [m, n], [k], order=abi.ORDER_DEVICE, name=b"dot+add" if add else b"dot")
        l.n_inputs, l.int_accum = 3 if add else 2, 1
        l.iparam[1] = abi.BF16
        l.inputs[0].dtype, l.inputs[0].affine, l.inputs[0].affine_zero, l.inputs[0].affine_scale = abi.I8, 1, int(dims[3]) if len(dims) > 3 else 0, 0.03125
        l.inputs[0].stride[0], l.inputs[0].stride[2], l.inputs[0].numel = k, 1, m * k
        l.inputs[1].dtype, l.inputs[1].stride[1], l.inputs[1].stride[2], l.inputs[1].numel = abi.I8, 1, n, k * n
        l.inputs[1].scale_stride[1] = 1
        l.out.dtype, l.out.stride[0], l.out.stride[1], l.out.numel = abi.BF16, n, 1, m * n
        table = [a, b, c, sw]
        if add:
            l.inputs[2].dtype, l.inputs[2].stride[0], l.inputs[2].stride[1], l.inputs[2].numel = abi.BF16, n, 1, m * n
            table = [a, b, ex.upload(bf16((m, n))), c, sw]
        ms = timed(lambda: ex.run(l, table), args.steps)
        print(json.dumps({"micro": "gemm_i8", "shape": dims, "ms": ms, "TOP/s": 2.0 * m * n * k / ms / 1e9}))
    elif args.micro == "contract":
        # x[m, k] · w[k, n] in bf16 as a contraction launch (what a model's projection issues): with a few rows the
        # executor cuts the summed axis into runs; the figure that matters then is the rate the weights stream at
        m, n, k = dims[:3]
        a, b = ex.upload(bf16((m, k))), ex.upload(bf16((k, n)))
        c = ex.alloc(m * n * 2)
        l = launch_desc(abi.OP_CONTRACT, abi.BF16, [m, n], [k], order=abi.ORDER_DEVICE, name=b"dot")
        l.n_inputs = 2
        l.inputs[0].dtype, l.inputs[0].stride[0], l.inputs[0].stride[2], l.inputs[0].numel = abi.BF16, k, 1, m * k
        l.inputs[1].dtype, l.inputs[1].stride[1], l.inputs[1].stride[2], l.inputs[1].numel = abi.BF16, 1, n, k * n
        l.out.dtype, l.out.stride[0], l.out.stride[1], l.out.numel = abi.BF16, n, 1, m * n
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if len(dims) > 3 and dims[3] else None  # 4th number 1: write 256 MB between calls, so that the weights come from HBM

        def once():
            if flush is not None:
                with torch.cuda.stream(stream):
                    flush.zero_()
            ex.run(l, [a, b, c])

        ex.set_profiling(True)
        ms = timed(once, args.steps)
        rows = ex.profile()
        ex.set_profiling(False)
        per = {}
        for rec in rows[-args.steps:]:
            per.setdefault(rec[0], []).append(rec[2])
        print(json.dumps({"micro": "contract", "shape": dims, "ms a call (with the flush, if any)": ms, "kernel ms": {k_: float(np.median(v)) for k_, v in per.items()}, "weights GB": 2.0 * k * n / 1e9,
                          "GB/s of the weights over the launch's kernels": 2.0 * k * n / 1e6 / sum(float(np.median(v)) for v in per.values())}))
    elif args.micro == "attn_step":
        # one new position against a cache: q [B, H, 1, 128], k [B, H, len, 128], v [B, len, H, 128]
        B, H, t = dims[:3]
        hd = 128
        q, k, v = ex.upload(bf16((B, H, 1, hd))), ex.upload(bf16((B, H, t, hd))), ex.upload(bf16((B, t, H, hd)))
        rt = ex.upload(np.array([0x4135], np.uint16))
        out = ex.alloc(B * H * hd * 2)
        l = launch_desc(abi.OP_ATTENTION, abi.BF16, [B, H, 1, hd], [t], order=abi.ORDER_DEVICE, name=b"attention[blockwise]")
        l.n_inputs = 4
        l.iparam[1] = l.iparam[2] = l.iparam[3] = abi.BF16
        for o, st, n in ((l.inputs[0], (H * hd, hd, 0, 1, 0), B * H * hd), (l.inputs[1], (H * t * hd, t * hd, 0, 1, hd), B * H * t * hd), (l.inputs[2], (t * H * hd, hd, 0, 1, H * hd), B * H * t * hd), (l.out, (H * hd, hd, 0, 1, 0), B * H * hd)):
            o.dtype, o.numel = abi.BF16, n
            for a, x in enumerate(st):
                o.stride[a] = x
        l.inputs[3].dtype, l.inputs[3].numel = abi.BF16, 1
        ms = timed(lambda: ex.run(l, [q, k, v, rt, out]), args.steps)
        print(json.dumps({"micro": "attn_step", "shape": dims, "ms": ms, "GB/s of the cache": 2.0 * 2.0 * B * H * t * hd / ms / 1e6}))
    elif args.micro == "attn":
        B, H, t = dims[:3]
        hd = 128
        q, k, v = ex.upload(bf16((B, H, t, hd))), ex.upload(bf16((B, H, t, hd))), ex.upload(bf16((B, t, H, hd)))
        rt = ex.upload(np.array([0x4135], np.uint16))  # bf16(sqrt(128)) = 11.3125
        out = ex.alloc(B * H * t * hd * 2)
        lm = launch_desc(abi.OP_IOTA, abi.F32, [t, t])
        lm.kind = abi.IOTA_CAUSAL
        lm.out.dtype, lm.out.is_index, lm.out.stride[0], lm.out.stride[1] = abi.I64, 1, t, 1
        mask = ex.alloc(t * t * 8)
        ex.run(lm, [mask])
        l = launch_desc(abi.OP_ATTENTION, abi.BF16, [B, H, t, hd], [t], order=abi.ORDER_DEVICE, name=b"attention[blockwise]")
        l.n_inputs, l.masked = 5, 1
        l.iparam[0] = dims[3] if len(dims) > 3 else 0  # 1: the one-pass kernel (`attention: online`)
        l.iparam[1] = l.iparam[2] = l.iparam[3] = abi.BF16
        n = B * H * t * hd
        for o, st in ((l.inputs[0], (H * t * hd, t * hd, hd, 1, 0)), (l.inputs[1], (H * t * hd, t * hd, 0, 1, hd)), (l.inputs[2], (t * H * hd, hd, 0, 1, H * hd)), (l.out, (t * H * hd, hd, H * hd, 1, 0))):
            o.dtype, o.numel = abi.BF16, n
            for a, x in enumerate(st):
                o.stride[a] = x
        l.inputs[3].dtype, l.inputs[3].numel = abi.BF16, 1
        if len(dims) > 4 and dims[4] == 1:  # 5th number 1: the result as i8 codes of a scaled site (the one-pass kernel only)
            l.out.dtype, l.out.affine, l.out.affine_zero, l.out.affine_scale = abi.I8, 1, 0, 0.02
        l.inputs[4].dtype, l.inputs[4].is_index, l.inputs[4].stride[2], l.inputs[4].stride[4], l.inputs[4].numel = abi.I64, 1, t, 1, t * t
        ms = timed(lambda: ex.run(l, [q, k, v, rt, mask, out]), args.steps)
        nqb = t // 128
        fl = 4.0 * B * H * (nqb * (nqb + 1) / 2) * 128 * 128 * hd
        print(json.dumps({"micro": "attn", "shape": dims, "ms": ms, "TFLOP/s (causal blocks, one pass)": fl / ms / 1e9}))
    elif args.micro == "f32c":
        # x[m, k] · w[k, n], every site f32, under the device order (three bf16 planes an operand)
        m, n, k = dims[:3]
        a, b = ex.upload(rng.standard_normal((m, k)).astype(np.float32)), ex.upload(rng.standard_normal((k, n)).astype(np.float32))
        c = ex.alloc(m * n * 4)
        l = launch_desc(abi.OP_CONTRACT, abi.F32, [m, n], [k], order=abi.ORDER_DEVICE if len(dims) < 4 or dims[3] else abi.ORDER_SEQUENTIAL)
        l.n_inputs = 2
        l.inputs[0].dtype, l.inputs[0].numel, l.inputs[0].stride[0], l.inputs[0].stride[2] = abi.F32, m * k, k, 1
        l.inputs[1].dtype, l.inputs[1].numel, l.inputs[1].stride[1], l.inputs[1].stride[2] = abi.F32, n * k, 1, n
        l.out.dtype, l.out.numel, l.out.stride[0], l.out.stride[1] = abi.F32, m * n, n, 1
        ms = timed(lambda: ex.run(l, [a, b, c]), args.steps)
        print(json.dumps({"micro": "f32c", "shape": dims, "ms": ms, "TFLOP/s (2mnk)": 2.0 * m * n * k / ms / 1e9}))
    elif args.micro == "e8m15":
        # the contraction-plus-LayerNorm workload's contraction: x[m, k] · w[k, n], every site e8m15, under the device order
        m, n, k = dims[:3]
        a = ex.upload(rng.integers(0, 256, size=m * k * 3, dtype=np.uint8) & np.tile(np.array([255, 255, 0x3f], np.uint8), m * k))
        b = ex.upload(rng.integers(0, 256, size=n * k * 3, dtype=np.uint8) & np.tile(np.array([255, 255, 0x3f], np.uint8), n * k))
        c = ex.alloc(m * n * 3)
        l = launch_desc(abi.OP_CONTRACT, abi.E8M15, [m, n], [k], order=abi.ORDER_DEVICE)
        l.n_inputs = 2
        l.inputs[0].dtype, l.inputs[0].numel, l.inputs[0].stride[0], l.inputs[0].stride[2] = abi.E8M15, m * k, k, 1
        l.inputs[1].dtype, l.inputs[1].numel, l.inputs[1].stride[1], l.inputs[1].stride[2] = abi.E8M15, n * k, 1, n
        l.out.dtype, l.out.numel, l.out.stride[0], l.out.stride[1] = abi.E8M15, m * n, n, 1
        ms = timed(lambda: ex.run(l, [a, b, c]), args.steps)
        print(json.dumps({"micro": "e8m15", "shape": dims, "ms": ms, "TFLOP/s (2mnk)": 2.0 * m * n * k / ms / 1e9}))
    elif args.micro == "norm":
        # a norm's last group: x[rows, n] / root[rows] (f32) * gamma[n]
        rows, n = dims[:2]
        x, gam = ex.upload(bf16((rows, n))), ex.upload(bf16((n,)))
        root = ex.upload((np.abs(rng.standard_normal(rows)) + 0.5).astype(np.float32))
        out = ex.alloc(rows * n * 2)
        l = launch_desc(abi.OP_FUSED, abi.BF16, [rows, n], order=abi.ORDER_DEVICE)
        l.n_inputs, l.n_steps = 3, 2
        l.steps[0].prim, l.steps[0].nargs, l.steps[0].src[0], l.steps[0].src[1] = abi.DIV, 2, 0, 1
        l.steps[1].prim, l.steps[1].nargs, l.steps[1].src[0], l.steps[1].src[1] = abi.MUL, 2, -1, 2
        for o in (l.inputs[0], l.out):
            o.dtype, o.stride[0], o.stride[1], o.numel = abi.BF16, n, 1, rows * n
        l.inputs[1].dtype, l.inputs[1].stride[0], l.inputs[1].numel = abi.F32, 1, rows
        l.inputs[2].dtype, l.inputs[2].stride[1], l.inputs[2].numel = abi.BF16, 1, n
        ms = timed(lambda: ex.run(l, [x, root, gam, out]), args.steps)
        print(json.dumps({"micro": "norm", "shape": dims, "ms": ms, "GB/s": rows * n * 4 / ms / 1e6}))
    elif args.micro == "rmsnorm":
        # the merged RMSNorm launch: x[rows, n] bf16, f32 statistics, gamma[n]; --shape rows,n[,s]: with a third
        # number the result is a scaled site's i8 codes with the scale s / 1000
        rows, n = dims[:2]
        x, gam = ex.upload(bf16((rows, n))), ex.upload(bf16((n,)))
        eps = ex.upload(np.array([1e-5], np.float32))
        out = ex.alloc(rows * n * 2)
        l = launch_desc(abi.OP_RMSNORM, abi.BF16, [rows, n], order=abi.ORDER_DEVICE, name=b"rmsnorm[merged]")
        l.n_inputs = 3
        l.iparam[0], l.iparam[1], l.iparam[2], l.iparam[3] = n, abi.BF16, abi.F32, abi.F32
        for o in (l.inputs[0], l.out):
            o.dtype, o.stride[0], o.stride[1], o.numel = abi.BF16, n, 1, rows * n
        l.inputs[1].dtype, l.inputs[1].numel = abi.F32, 1
        l.inputs[2].dtype, l.inputs[2].stride[1], l.inputs[2].numel = abi.BF16, 1, n
        codes = len(dims) > 2 and dims[2] > 0
        if codes:
            l.out.dtype, l.out.affine, l.out.affine_zero, l.out.affine_scale = abi.I8, 1, 0, dims[2] / 1000.0
        ms = timed(lambda: ex.run(l, [x, eps, gam, out]), args.steps)
        print(json.dumps({"micro": "rmsnorm", "shape": dims, "ms": ms, "GB/s": rows * n * (3 if codes else 4) / ms / 1e6}))
    elif args.micro == "rope":
        # the merged rotation: x[rows, seq, 2, rot] bf16 with cos and sin over [seq, rot]; --shape rows,seq,rot
        rows, seq, rot = dims[:3]
        x, c, sn = ex.upload(bf16((rows, seq, 2, rot))), ex.upload(bf16((seq, rot))), ex.upload(bf16((seq, rot)))
        n = rows * seq * 2 * rot
        out = ex.alloc(n * 2)
        l = launch_desc(abi.OP_ROPE, abi.BF16, [rows, seq, 2, rot], order=abi.ORDER_DEVICE, name=b"rope[merged]")
        l.n_inputs = 3
        for o in (l.inputs[0], l.out):
            o.dtype, o.numel = abi.BF16, n
            o.stride[0], o.stride[1], o.stride[2], o.stride[3] = seq * 2 * rot, 2 * rot, rot, 1
        for o in (l.inputs[1], l.inputs[2]):
            o.dtype, o.numel, o.stride[1], o.stride[3] = abi.BF16, seq * rot, rot, 1
        ms = timed(lambda: ex.run(l, [x, c, sn, out]), args.steps)
        print(json.dumps({"micro": "rope", "shape": dims, "ms": ms, "GB/s": n * 4 / ms / 1e6}))
    elif args.micro == "xent":
        # cross-entropy of f32 logits [rows, v] against labels, under the device order; --shape rows,v
        rows, v = dims[:2]
        x = ex.upload(rng.standard_normal((rows, v)).astype(np.float32))
        y = ex.upload(rng.integers(0, v, size=(rows,), dtype=np.int64))
        out = ex.alloc(rows * 4)
        l = launch_desc(abi.OP_XENT, abi.F32, [rows], [v], order=abi.ORDER_DEVICE, name=b"cross_entropy")
        l.n_inputs = 2
        l.inputs[0].dtype, l.inputs[0].numel, l.inputs[0].stride[0], l.inputs[0].stride[1] = abi.F32, rows * v, v, 1
        l.inputs[1].dtype, l.inputs[1].is_index, l.inputs[1].numel, l.inputs[1].stride[0] = abi.I64, 1, rows, 1
        l.out.dtype, l.out.numel, l.out.stride[0] = abi.F32, rows, 1
        ms = timed(lambda: ex.run(l, [x, y, out]), args.steps)
        print(json.dumps({"micro": "xent", "shape": dims, "ms": ms, "GB/s": rows * v * 4 / ms / 1e6}))
    elif args.micro in ("softmax", "ew"):
        rows, n = dims[:2]
        x = ex.upload(bf16((rows, n)))
        out = ex.alloc(rows * n * 2)
        if args.micro == "softmax":
            t = n  # rows are (batch·heads, seq): the causal mask is [n, n]
            lm = launch_desc(abi.OP_IOTA, abi.F32, [t, t])
            lm.kind = abi.IOTA_CAUSAL
            lm.out.dtype, lm.out.is_index, lm.out.stride[0], lm.out.stride[1] = abi.I64, 1, t, 1
            mask = ex.alloc(t * t * 8)
            ex.run(lm, [mask])
            l = launch_desc(abi.OP_SOFTMAX, abi.BF16, [rows // t, t], [n], order=abi.ORDER_DEVICE)
            l.n_inputs, l.masked = 2, 1
            for o in (l.inputs[0], l.out):
                o.dtype, o.stride[0], o.stride[1], o.stride[2], o.numel = abi.BF16, t * n, n, 1, rows * n
            l.inputs[1].dtype, l.inputs[1].is_index, l.inputs[1].stride[1], l.inputs[1].stride[2], l.inputs[1].numel = abi.I64, 1, n, 1, t * t
            ms = timed(lambda: ex.run(l, [x, mask, out]), args.steps)
        else:
            l = launch_desc(abi.OP_FUSED, abi.BF16, [rows, n], order=abi.ORDER_DEVICE)
            l.n_inputs, l.n_steps = 2, 1
            l.steps[0].prim, l.steps[0].nargs, l.steps[0].src[0], l.steps[0].src[1] = abi.ADD, 2, 0, 1
            for o in (l.inputs[0], l.inputs[1], l.out):
                o.dtype, o.stride[0], o.stride[1], o.numel = abi.BF16, n, 1, rows * n
            ms = timed(lambda: ex.run(l, [x, x, out]), args.steps)
        traffic = rows * n * 2 * (2 if args.micro == "softmax" else 3)
        print(json.dumps({"micro": args.micro, "shape": dims, "ms": ms, "GB/s": traffic / ms / 1e6}))


def load_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        return {}


def profile_table(rows):
    """{kernel family: [launches, ms, flops, algorithmic bytes]} of psk_exec_profile's rows."""
    by = {}
    for k, name, kms, fl, bts in rows:
        d = by.setdefault(k, [0, 0.0, 0.0, 0.0])
        d[0] += 1; d[1] += kms; d[2] += fl; d[3] += bts
    return by


def shares_of(by):
    total = sum(d[1] for d in by.values()) or 1.0
    return {k: {"launches": d[0], "ms": round(d[1], 3), "share": round(d[1] / total, 4), "GB/s": round(d[3] / (d[1] * 1e-3) / 1e9, 1) if d[1] > 0 else None} for k, d in sorted(by.items(), key=lambda kv: -kv[1][1])}


# ---- the smaller configurations --------------------------------------------------------------------------------
def small_case(name, w):
    """(model, consts, realization, params, inputs of `entry`, entry, units a step, unit, flops a step) of a small workload."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import models
    if w["kind"] == "mlp":
        B = w["B"]
        x, y = models.mlp_inputs(B)
        return dict(model="mlp", consts={}, rz="f32", params=models.mlp_params(), inputs=[x, y], entry="loss", units=B, unit="samples/s",
                    metric="samples/sec 2-layer ReLU MLP forward+loss", flops=2.0 * B * (784 * 256 + 256 * 10), dtype="f32", order="sequential")
    if w["kind"] == "gpt":
        c, B, T = w["consts"], w["B"], w["T"]
        rng = np.random.default_rng(2)
        ids = rng.integers(0, c["V"], size=(B, T), dtype=np.int64)
        y = rng.integers(0, c["V"], size=(B, T), dtype=np.int64)
        rz = {"default": "bf16", "order": {"kind": "device"}, "storage": {"LayerNorm.apply/%2": "f32", "LayerNorm.apply/%5": "f32", "LayerNorm.apply/%10": "f32", "GPT.apply/%24": "f32", "loss/%6": "f32", "loss/%7": "f32"}}
        D, L, V = c["D"], c["L"], c["V"]
        return dict(model="gpt", consts=c, rz=rz, params=models.gpt_params(c, T), inputs=[ids, y], entry="loss", units=B * T, unit="tokens/s",
                    metric="tokens/sec small GPT forward+loss", flops=float(B * T) * (L * (24 * D * D + 4 * T * D) + 2 * D * V), dtype="bf16 storage, f32 accumulation", order="device")
    n, dt = w["N"], w["dtype"]
    rng = np.random.default_rng(n)
    x = rng.standard_normal((n, n), dtype=np.float32)
    wt = rng.standard_normal((n, n), dtype=np.float32)
    rz = {"default": dt, "order": {"kind": "device"}}
    if dt == "f16" and n >= 4096:
        # a row of x·w has deviations of about sqrt(n) a term, so the squared deviations of LayerNorm pass binary16's
        # largest number (65504) from n = 4096 on and the all-f16 program stops with E7007, as the reference's does;
        # those two sites are kept in f32 here (what a solved realization would do), everything else stays binary16
        rz["storage"] = {"LayerNorm.apply/%5": "f32", "LayerNorm.apply/%6": "f32"}  # and their mean, which an f16 kernel would round at its edge
    return dict(model="contract_ln", consts={}, rz=rz, params={"ln.γ": np.ones(n, np.float32), "ln.β": np.zeros(n, np.float32)}, inputs=[x, wt], entry="apply",
                units=2.0 * n * n * n / 1e12, unit="TFLOP/s", metric=f"TFLOP/s (2·N^3) of x·w + row LayerNorm, N={n}, stored {dt}", flops=2.0 * n * n * n, dtype=f"{dt} storage, f32 accumulation", order="device", out_shape=(n, n))


def small_cpu(case, w, threads):
    """The CPU restatement on the same inputs at full size (a bounded part of the rows for the largest contraction)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import models
    import oracle_lib
    from presk_b200 import Host
    os.environ["OMP_NUM_THREADS"] = str(threads)
    orc = oracle_lib.load()
    rz = case["rz"] if isinstance(case["rz"], str) else dict(case["rz"], order={"kind": "sequential"})
    h = models.give(Host(orc.vtable(), rz).prepare(case["model"], **case["consts"]), case["params"])
    inputs, frac, note = case["inputs"], 1.0, "full size"
    if w["kind"] == "contract_ln" and w["N"] > 4096:
        rows = 256  # every row of x is an independent 1/N of the work (its row of the product, its LayerNorm)
        inputs = [np.ascontiguousarray(inputs[0][:rows]), inputs[1]]
        frac, note = rows / w["N"], f"{rows} of the {w['N']} rows of x (rows are independent; time scaled by {w['N'] // rows})"
    out_shape = case.get("out_shape", ())
    if out_shape and frac < 1.0:
        out_shape = (inputs[0].shape[0], out_shape[1])
    med, raw = time_call(lambda: h.call(case["entry"], inputs, out_shape), warmup=1, reps=3)
    h.close()
    value = case["units"] / (med / frac)
    return value, f"oracle (C restatement, OpenMP, {threads} threads), {note}; warm-up 1 + median of 3: [" + ", ".join(f"{t:.3f}" for t in raw) + "] s"


def run_small(args, name, w):
    threads = os.cpu_count() or 1
    rank = int(os.environ.get("RANK", 0))
    case = small_case(name, w)
    config = {"workload": name, **{k: v for k, v in w.items() if k != "kind"}, "realization": case["rz"] if isinstance(case["rz"], str) else json.dumps(case["rz"], ensure_ascii=False), "l2": "flushed between timed steps (a 256 MB buffer is overwritten)", "parallelism": "replicas (one GPU holds the whole problem)"}
    if args.impl == "reference":
        if rank != 0:
            return
        v, sample = small_cpu(case, w, threads)
        print(json.dumps({"impl": "reference", "metric": case["metric"], "value": v, "unit": case["unit"], "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * case["units"] / v,
                          "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": case["dtype"], "data": "synthetic", "config": config,
                          "cpu_baseline": {"value": v, "unit": case["unit"], "cores": threads, "kind": "port", "sample": sample}, "e2e": {"value": v, "unit": case["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import models
    from presk_b200 import Executor, Host, abi
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    ex = Executor(local)
    host = models.give(Host(ex, case["rz"]).prepare(case["model"], **case["consts"]), case["params"])
    stream = torch.cuda.ExternalStream(ex.stream(), device=torch.device("cuda", local))
    dev_inputs = []
    for a in case["inputs"]:
        dev_inputs.append((ex.upload(a), abi.I64 if a.dtype == np.int64 else abi.F32, a.shape))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=f"cuda:{local}")
    warm = max(args.warmup, 3)
    for _ in range(warm):
        host.call_device(case["entry"], dev_inputs)
    ex.sync()
    _, k0 = ex.counts()
    sampler = ClockSampler(local)
    sampler.start()
    ms = 0.0
    evs = []
    for _ in range(args.steps):
        with torch.cuda.stream(stream):
            flush.zero_()  # L2 holds nothing of the step before
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        host.call_device(case["entry"], dev_inputs)
        e1.record(stream)
        evs.append((e0, e1))
    ex.sync()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = sum(a.elapsed_time(b) for a, b in evs)
    _, k1 = ex.counts()
    # the kernels' shares from a pass of its own: events around every launch cost a launch-bound step more than they tell
    ex.set_profiling(True)
    for _ in range(args.steps):
        host.call_device(case["entry"], dev_inputs)
    rows = ex.profile()
    ex.set_profiling(False)
    # end to end: host arrays in, the result read back, every step
    out_shape = case.get("out_shape", ())
    for _ in range(2):
        host.call(case["entry"], case["inputs"], out_shape)
    ex.sync()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        res = host.call(case["entry"], case["inputs"], out_shape)
    ex.sync()
    e2e_s = time.perf_counter() - t0
    by = profile_table(rows)
    peaks = load_peaks()
    hbm_peak = peaks.get("hbm_gbs") or 6650.0
    tf_peak = peaks.get("bf16_tflops") or 1590.0
    top = max(by.items(), key=lambda kv: kv[1][1]) if by else ("none", [0, 0.0, 0.0, 0.0])
    if top[0] == "k_gemm_tc":
        ach = top[1][2] / (top[1][1] * 1e-3) / 1e12
        roof = {"bound": "tensor", "kernel": top[0], "achieved": ach, "peak": tf_peak, "unit": "TFLOP/s", "frac": ach / tf_peak, "traffic": None}
    else:
        ach = top[1][3] / (top[1][1] * 1e-3) / 1e9 if top[1][1] > 0 else 0.0
        roof = {"bound": "hbm", "kernel": top[0], "achieved": ach, "peak": hbm_peak, "unit": "GB/s", "frac": ach / hbm_peak, "traffic": None}
    roof["peak_source"] = "measured (MEASURED_PEAKS.json: copy bandwidth, burst cuBLAS bf16)" if peaks else "fallback"
    roof["note"] = "algorithmic work of the kernel family with the largest share of the step, over its event-timed launches"
    out = {"metric": case["metric"], "value": case["units"] * args.steps / (ms * 1e-3), "unit": case["unit"], "n_gpus": 1, "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps,
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": case["dtype"], "data": "synthetic", "config": config,
           "e2e": {"value": case["units"] * args.steps / e2e_s, "unit": case["unit"], "h2d_bytes_per_step": int(sum(a.nbytes for a in case["inputs"])), "d2h_bytes_per_step": int(np.asarray(res).nbytes)},
           "gpu_launches": int(k1 - k0), "clocks": clocks, "roofline": roof, "kernel_shares": shares_of(by), "model_tflops": case["flops"] * args.steps / (ms * 1e-3) / 1e12}
    if not args.no_cpu_baseline:
        try:
            v, sample = small_cpu(case, w, threads)
            out["cpu_baseline"] = {"value": v, "unit": case["unit"], "cores": threads, "kind": "port", "sample": sample}
        except Exception as e:  # the baseline is reported, never the product's path
            out["cpu_baseline"] = {"value": None, "unit": case["unit"], "cores": threads, "kind": "port", "sample": f"failed: {e}"}
    print(json.dumps(out, ensure_ascii=False))


def run_decode(args, name, w):
    """Generation with a key/value cache: `prefill` once (untimed), then timed `step` calls, one new token a sequence."""
    consts, B, T = w["consts"], w["B"], w["T"]
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    threads = os.cpu_count() or 1
    warm = max(args.warmup, 3)
    tmax = T + warm + 3 * args.steps + 8
    config = {"workload": name, **consts, "batch_per_gpu": B, "context": T, "global_batch": B * world, "parallelism": f"dp{world} (sequences are independent: no collective)",
              "realization": "bf16 storage, f32 norm statistics/logits, order device, launches merged; keys and values cached per layer",
              "l2": "inputs_larger_than_l2 (13.5 GB of weights and the cache stream through every step)"}
    D, FF, L, V, H = consts["D"], consts["FF"], consts["L"], consts["V"], consts["H"]
    if args.impl == "reference":
        if rank != 0:
            return
        # the reference has no cache: a new token costs a whole window's prefill (presk-serve/src/lib.rs:241)
        v, sample = cpu_prefill_tokens_per_s(consts, T, 1, threads, False, direct=True)
        val = v / (T + 1)
        print(json.dumps({"impl": "reference", "metric": "generated tokens/sec Llama-7B-shape decode", "value": val, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                          "ms_per_step": 1e3 * B / val, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 storage, f32 arithmetic", "data": "synthetic", "config": config,
                          "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": "one generated token = one whole window recomputed, as the reference's serve loop does (no cache): prefill rate / (context + 1); " + sample},
                          "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    import torch
    import torch.distributed as dist
    from presk_b200 import Executor, Host, abi, shard
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ex = Executor(local)
    shapes = param_shapes(consts)
    host = Host(ex, realization(shapes, False, "blockwise", "merged")).prepare("llama", TMAX=tmax, **consts)
    for i, (path, (shape, std)) in enumerate(shapes.items()):
        host.init_param(path, 1000 + i, std, shape)
    rng = np.random.default_rng(rank)
    ids = rng.integers(0, V, size=(B, T), dtype=np.int64)
    nxt = rng.integers(0, V, size=(B, 1), dtype=np.int64)
    host.call("prefill", [ids], (B, T, V))
    nxt_dev = ex.upload(nxt)
    dev_in = [(nxt_dev, abi.I64, (B, 1))]
    stream = torch.cuda.ExternalStream(ex.stream(), device=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        ex.sync()
        torch.cuda.synchronize()

    for _ in range(warm):
        host.call_device("step", dev_in)
    ex.sync()
    _, k0 = ex.counts()
    l0 = ex.counts()[0]
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        host.call_device("step", dev_in)
    e1.record(stream)
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    l1, k1 = ex.counts()
    # the per-kernel times come from a pass of their own: a pair of events around each of several hundred launches
    # of microseconds would be most of the timed region
    ex.set_profiling(True)
    for _ in range(args.steps):
        host.call_device("step", dev_in)
    ex.sync()
    rows = ex.profile()
    ex.set_profiling(False)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        logits = host.call("step", [nxt], (B, 1, V))
    barrier()
    e2e_s = time.perf_counter() - t0
    ms = shard.max_over_ranks(ms, device="cuda")
    e2e_ms = shard.max_over_ranks(e2e_s * 1e3, device="cuda")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    peaks = load_peaks()
    hbm_peak = peaks.get("hbm_gbs") or 6650.0
    by = profile_table(rows)
    # what a step must read: every weight once, and the cache's keys and values of the positions so far
    ctx_mid = T + warm + args.steps / 2.0
    weight_bytes = 2.0 * (L * (4 * D * D + 3 * D * FF) + D * V)
    cache_bytes = 2.0 * 2.0 * L * B * ctx_mid * D
    achieved = (weight_bytes + cache_bytes) * args.steps / (ms * 1e-3) / 1e9
    tokens = B * world * args.steps
    out = {"metric": "generated tokens/sec Llama-7B-shape decode", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps,
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 storage, f32 accumulation", "data": "synthetic", "config": config,
           "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": int(nxt.nbytes), "d2h_bytes_per_step": int(logits.nbytes)},
           "gpu_launches": int(k1 - k0), "launches_per_step": int((l1 - l0) / args.steps), "clocks": clocks,
           "roofline": {"bound": "hbm", "kernel": "the whole step (weights and cache read once)", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak, "traffic": None,
                        "algorithmic_bytes_per_step": weight_bytes + cache_bytes, "peak_source": "measured (MEASURED_PEAKS.json, copy bandwidth)" if peaks else "fallback",
                        "kernel_ms_per_step": sum(d[1] for d in by.values()) / args.steps},
           "kernel_shares": shares_of(by)}
    if world == 1 and not args.no_cpu_baseline:
        try:
            v, sample = cpu_prefill_tokens_per_s(consts, T, 1, threads, False)
            out["cpu_baseline"] = {"value": v / (T + 1), "unit": "tokens/s", "cores": threads, "kind": "port", "sample": "one generated token = one whole window recomputed, as the reference's serve loop does (no cache): prefill rate / (context + 1); " + sample}
        except Exception as e:
            out["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": f"failed: {e}"}
    print(json.dumps(out, ensure_ascii=False))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--micro", default=None, choices=["gemm", "gemm_i8", "contract", "softmax", "ew", "attn", "attn_step", "norm", "e8m15", "f32c", "train", "rmsnorm", "rope", "xent"])
    ap.add_argument("--shape", default="8192,8192,8192")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama7b_prefill_b8_t2048", choices=sorted(WORKLOADS))
    ap.add_argument("--attention", default="online", choices=["blockwise", "online", "unfused"], help="the declared order of the attention launches: one kernel in two passes over the keys (blockwise) or in one (online), or the reference's four launches")
    ap.add_argument("--launches", default="merged", choices=["merged", "reference"], help="merged: bit-preserving rewrites of the launch list (views for slices, in-place concatenation, wider groups); reference: the reference's launch list")
    ap.add_argument("--comm", default="psk", choices=["psk", "torch"], help="what carries the loss gather of a sharded run: the library's psk_comm_* (NCCL on the executor's stream) or torch.distributed")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the parity pre-flight against the CPU oracle")
    ap.add_argument("--dump-profile", default=None, help="write the per-launch-name times of the timed steps to this file")
    args = ap.parse_args()
    if args.micro:
        return microbench(args)
    w = WORKLOADS[args.workload]
    if w.get("kind") == "decode":
        return run_decode(args, args.workload, w)
    if w.get("kind", "llama") != "llama":
        return run_small(args, args.workload, w)
    consts, B, T = w["consts"], w["B"], w["T"]
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    threads = os.cpu_count() or 1
    config = {"workload": args.workload, **{k: v for k, v in consts.items()}, "batch_per_gpu": B, "seq_len": T, "global_batch": B * world, "parallelism": f"dp{world}", "realization": "bf16 storage, f32 norm statistics/logits/loss, order device, attention " + args.attention + ", launches " + args.launches
              + {True: "; projection and FFN weights int8 with a scale a channel", "e4m3fn": "; projection and FFN weights stored e4m3fn",
                 "w8a8": "; W8A8: the projections' inputs as i8 codes with static scales from a calibration pass, projection, FFN and head weights int8, those contractions' products and sums i32; the attention's result "
                         + ("in i8 codes as well (all seven projections integer sums)" if w8a8_attention_in_codes(args.attention, args.launches) else "bf16 (the out-projection reads it against widened weights)")}.get(w.get("int8", False), ""),
              "l2": "inputs_larger_than_l2 (the weights stream through every step)"}

    if args.impl == "reference":
        if rank != 0:
            return
        v, sample = cpu_prefill_tokens_per_s(consts, T, B, threads, w.get("int8", False), direct=True)
        print(json.dumps({
            "impl": "reference", "metric": "tokens/sec Llama-7B-shape prefill", "value": v, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 * B * T / v, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 storage, f32 arithmetic", "data": "synthetic",
            "config": config, "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference's Rust executors cannot be built on this box (no cargo/rustc); this is the C restatement of the same loop nests (oracle/), OpenMP over the host's cores; a step is a bounded sample (one layer of the full width at the workload's sequence length, one sequence) and ms_per_step is the extrapolation to the whole depth and batch",
        }))
        return

    import torch
    import torch.distributed as dist
    from presk_b200 import Comm, Executor, Host, abi, shard

    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ex = Executor(local)
    comm, comm_kind = None, "none (one rank)"
    if world > 1:
        comm_kind = "torch.distributed (NCCL)"
        if args.comm == "psk":
            # rank 0 makes the communicator's id; the others get it over the process group that started them
            box = [Comm.unique_id() if rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            try:
                comm = Comm(ex, world, rank, box[0])
                comm_kind = "psk_comm (NCCL on the executor's stream)"
            except Exception as e:  # reported in the line; the gather then goes through torch.distributed
                comm_kind = f"torch.distributed (psk_comm could not be made: {e})"
            # every rank must take the same route
            flags = torch.tensor([1.0 if comm is not None else 0.0], device="cuda")
            dist.all_reduce(flags, op=dist.ReduceOp.MIN)
            if float(flags[0]) == 0.0 and comm is not None:
                comm.close()
                comm = None
                comm_kind = "torch.distributed (psk_comm failed on another rank)"
    shapes = param_shapes(consts)
    rng = np.random.default_rng(rank)
    ids_pinned = torch.from_numpy(rng.integers(0, consts["V"], size=(B, T), dtype=np.int64)).pin_memory()
    y_pinned = torch.from_numpy(rng.integers(0, consts["V"], size=(B, T), dtype=np.int64)).pin_memory()
    ids_np, y_np = ids_pinned.numpy(), y_pinned.numpy()
    ids_dev, y_dev = ex.upload(ids_np), ex.upload(y_np)
    dev_inputs = [(ids_dev, abi.I64, (B, T)), (y_dev, abi.I64, (B, T))]
    w8a8_scales = None
    if w.get("int8") == "w8a8":
        # `presk calibrate` then `presk scales`: one pass of the bf16 realization with every launch's magnitudes
        # folded into its site (all ranks' merged), and an absmax scale a scaled site from them; outside every
        # timed region
        cal = Host(ex, realization(shapes, False, "unfused", "reference")).prepare("llama", **consts)
        for i, (path, (shape, std)) in enumerate(shapes.items()):
            cal.init_param(path, 1000 + i, std, shape)
        cal.set_calibrating(True)
        cal.call_device("loss", dev_inputs)
        ex.sync()
        if comm is not None:
            cal.envelope_allreduce(comm)
        env = cal.envelope()
        cal.close()
        w8a8_scales = {site: float(np.float32(env[site][0]) / np.float32(127.0)) for site in W8A8_SCALED + (W8A8_ATTN_OUT_SITE,)}
        host = Host(ex, w8a8_realization(shapes, args.attention, args.launches, w8a8_scales)).prepare("llama", **consts)
    else:
        host = Host(ex, realization(shapes, w.get("int8", False), args.attention, args.launches)).prepare("llama", **consts)
    for i, (path, (shape, std)) in enumerate(shapes.items()):
        host.init_param(path, 1000 + i, std, shape)
    ex.sync()
    stream = torch.cuda.ExternalStream(ex.stream(), device=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        ex.sync()
        torch.cuda.synchronize()

    def step_device():
        return host.call_device("loss", dev_inputs)

    for _ in range(max(args.warmup, 3)):
        step_device()
    ex.sync()
    launches_before, kernels_before = ex.counts()

    # ---- value: inputs resident, events on the executor's stream ----
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    ex.set_profiling(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        out_ptr, _, _ = step_device()
    e1.record(stream)
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    rows = ex.profile()
    ex.set_profiling(False)
    launches_after, kernels_after = ex.counts()

    # ---- e2e: host buffers in, the loss of the whole batch out, every step ----
    def step_e2e():
        if comm is not None:
            # all through the C ABI: two copies from pinned host memory, the launches, one all-reduce of the
            # per-rank mean on the executor's stream, the result read back
            ex._check(ex.lib.psk_exec_upload(ex.handle, ids_dev, ids_np.ctypes.data, ids_np.nbytes))
            ex._check(ex.lib.psk_exec_upload(ex.handle, y_dev, y_np.ctypes.data, y_np.nbytes))
            ptr, dt, _ = host.call_device("loss", dev_inputs)
            return host.mean_over_ranks(comm, ptr, dt)
        mine = float(host.call("loss", [ids_np, y_np], ()))
        return shard.combine_mean(mine, B * T, device="cuda") if world > 1 else mine

    for _ in range(2):
        step_e2e()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        loss_all = step_e2e()
    barrier()
    e2e_s = time.perf_counter() - t0

    ms = shard.max_over_ranks(ms, device="cuda")
    e2e_ms = shard.max_over_ranks(e2e_s * 1e3, device="cuda")
    tokens = B * T * world * args.steps
    value = tokens / (ms * 1e-3)
    e2e = tokens / (e2e_ms * 1e-3)
    if comm is not None:
        comm.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return

    peaks = load_peaks()
    tf_peak = peaks.get("bf16_tflops_sustained") or 1400.0
    hbm_peak = peaks.get("hbm_gbs") or 6650.0
    peak_kind = "measured (MEASURED_PEAKS.json, sustained cuBLAS bf16)" if peaks else "fallback"
    by = profile_table(rows)
    total_kernel_ms = sum(d[1] for d in by.values()) or 1.0
    if args.dump_profile:
        names = {}
        for k, name, kms, fl, bts in rows:
            # launches of one name and different sizes (a norm's scalar root and its scaling of a whole tensor) apart
            d = names.setdefault(k + " | " + name + f" | {bts / 1e6:.1f} MB", [0, 0.0, 0.0, 0.0])
            d[0] += 1; d[1] += kms; d[2] += fl; d[3] += bts
        with open(args.dump_profile, "w") as f:
            f.write("kernel | launch name | algorithmic bytes a launch\tlaunches\ttotal ms\tshare\tms/launch\tGB/s (algorithmic)\tTFLOP/s\n")
            for key, d in sorted(names.items(), key=lambda kv: -kv[1][1]):
                f.write(f"{key}\t{d[0]}\t{d[1]:.3f}\t{d[1] / total_kernel_ms:.4f}\t{d[1] / d[0]:.4f}\t{d[3] / (d[1] * 1e-3) / 1e9:.1f}\t{d[2] / (d[1] * 1e-3) / 1e12:.1f}\n")
    roof_kernel = "k_gemm_i8" if w.get("int8") == "w8a8" else "k_gemm_tc"
    tc = by.get(roof_kernel, [0, 0.0, 0.0, 0.0])
    achieved = tc[2] / (tc[1] * 1e-3) / 1e12 if tc[1] > 0 else 0.0
    if roof_kernel == "k_gemm_i8":
        # no 8-bit rate was measured on this pool: twice the measured bf16 rate, the nominal ratio of the two kinds
        tf_peak, peak_kind = 2.0 * tf_peak, "2 x " + peak_kind + " (the 8-bit kind's nominal ratio to bf16; integer operations, not FLOP)"
    out = {
        "metric": "tokens/sec Llama-7B-shape prefill", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 storage, f32 accumulation", "data": "synthetic",
        "config": config,
        "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": int(ids_np.nbytes + y_np.nbytes), "d2h_bytes_per_step": 8 if comm is not None else 4, "loss_gather": comm_kind},
        "gpu_launches": int(kernels_after - kernels_before),
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": roof_kernel, "achieved": achieved, "peak": tf_peak, "unit": "TFLOP/s", "frac": achieved / tf_peak, "traffic": GEMM_TRAFFIC.get(args.workload), "traffic_of": GEMM_TRAFFIC_OF if args.workload in GEMM_TRAFFIC else None, "peak_source": peak_kind,
                     "model_tflops": flops_per_token(consts, T) * B * T * args.steps / (ms * 1e-3) / 1e12, "hbm_peak_gbs": hbm_peak},
        "kernel_shares": shares_of(by),
        "loss": loss_all,
        "launches_per_step": int((launches_after - launches_before) / args.steps),
        "device_memory_gb": {"live": ex.memory()[0] / 1e9, "peak": ex.memory()[1] / 1e9},  # the executor's buffers, bf16 copies of narrow weights included
    }
    if not args.no_parity:
        out["parity"] = parity_preflight(ex, consts, w.get("int8", False), args.attention, args.launches)
    if world == 1 and not args.no_cpu_baseline:
        try:
            v, sample = cpu_prefill_tokens_per_s(consts, T, B, threads, w.get("int8", False))
            out["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample}
        except Exception as e:  # the baseline is reported, never the product's path
            out["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": f"failed: {e}"}
    print(json.dumps(out, ensure_ascii=False))


def parity_preflight(ex, consts, int8, attention="blockwise", launches="merged"):
    """Outside every timed region: one layer of the workload's own width (and its vocabulary) at B = 1, T = 256
    over the CUDA executor under the benchmark's realization and over the CPU oracle under the sequential order
    with the reference's launch list; the oracle is the checker. The largest difference of the logits against
    their scale, and both losses."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    try:
        import headline
        import oracle_lib
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
        weights = "int8" if int8 is True else (int8 if int8 in ("e4m3fn", "w8a8") else "bf16")
        if weights == "w8a8" and w8a8_attention_in_codes(attention, launches):
            weights = "w8a8_attn_out"
        r = headline.llama_width_parity(ex, oracle_lib.load(), B=1, T=256, weights=weights, consts={k: v for k, v in consts.items() if k != "L"}, order={"kind": "device", "attention": attention, "launches": launches})
        # (a value that crosses a code's boundary moves by a whole step of its i8 site: a wider bound a quantised site more)
        tol = headline.LOGITS_TOL * {"bf16": 1.0, "w8a8_attn_out": 4.0}.get(weights, 2.0) * r["logits_scale"]
        ok = r["finite"] and r["logits_max_err"] <= tol and abs(r["loss_gpu"] - r["loss_oracle"]) <= headline.LOSS_RTOL * abs(r["loss_oracle"])
        return {"ok": bool(ok), "max_err": r["logits_max_err"], "tol": tol, "mean_err": r["logits_mean_err"], "logits_scale": r["logits_scale"], "loss_gpu": r["loss_gpu"], "loss_oracle": r["loss_oracle"], "loss_rtol": headline.LOSS_RTOL,
                "shape": r["shape"], "against": f"CPU oracle, order sequential, the reference's launch list; the GPU side runs the benchmark's realization (device order, attention {attention}, launches {launches})"}
    except Exception as e:
        return {"ok": False, "error": str(e)}


if __name__ == "__main__":
    main()
