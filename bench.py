#!/usr/bin/env python
"""Benchmark of the lightning-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload C2|C3|C4|C4v|C5] [--no-secondary]

One "step" is one pass of the hot path over one batch of synthetic input.  The headline workload
is configuration 2 (lasd forward + backward, bf16, B=8 N=8192 H=32 D=E=128, per-head decay, fp32
initial state).  With N > 1 GPUs (torchrun, one rank per GPU) every rank runs its own batch of the
same shape -- the (batch, head) pairs are independent recurrences, so there is no data-path
collective -- and the reported value is the total over ranks divided by the slowest rank's time
(weak scaling).

Rank 0 prints ONE JSON line.  `value` is timed with inputs resident in HBM; `e2e` repeats the
measurement through the public Python API with pinned HOST buffers, host->device copies of all
inputs and device->host copies of all outputs inside the timed region.  `roofline` is for the
dominant kernel (HBM fraction on algorithmic bytes, plus the tensor-pipe fraction on algorithmic
flops), `cpu_baseline` times the CPU oracle (a port of the reference's torch operators) on a
bounded slice of the same workload on the host cores.  `secondary` carries the other
configurations of the metric, each with its own timing, roofline and a parity figure against the
CPU oracle on a slice of what was just computed: C3 (lavd fwd+bwd), C4 (64-step decode loop,
scalar and vector decay, GB/s) and C5 (1M-token packed stream; sequence-sharded over the ranks when
N > 1, together with the one-GPU time of the same stream measured in the same job).

--impl reference times the reference's own CPU algorithm (the oracle port under oracle/; the
reference checkout itself does not travel to the GPU box) on the same configuration.  It imports
no native code of this repository.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def traffic_table():
    """DRAM bytes per token-head per launch from the ncu captures summarised under profiles/
    (profiles/traffic.json, written next to each capture); empty if the file is missing."""
    p = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(p):
        return {}
    with open(p) as f:
        return json.load(f)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, val in zip(names, f[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


# --------------------------------------------------------------------------------------------
# workloads
# --------------------------------------------------------------------------------------------
def base_name(name):
    return "C4" if name == "C4v" else name


def make_workload(name, rank, world, dev, shape=None):
    """Inputs of one configuration.  Returns (cfg, inputs, tokens, algorithmic bytes, flops)."""
    from xopes_b200 import workloads as W
    cfg = dict(W.CONFIGS[base_name(name)])
    if shape and name != "C5":  # smaller case of the same kernel, for profiler captures
        b, n, h = (int(x) for x in shape.split(","))
        cfg.update(B=b, N=n, H=h) if base_name(name) != "C4" else cfg.update(B=b, H=h)
    seed = rank  # every rank draws its own batch
    flops = 0
    if name == "C2":
        w = W.lasd_inputs(cfg["B"], cfg["N"], cfg["H"], cfg["D"], cfg["E"], torch.bfloat16, seed)
        tokens = cfg["B"] * cfg["N"]
        alg_bytes = tokens * cfg["H"] * (W.BYTES_LASD_FWD + W.BYTES_LASD_BWD)
        flops = tokens * cfg["H"] * (W.FLOP_FWD + W.FLOP_BWD)
    elif name == "C3":
        w = W.lavd_inputs(cfg["B"], cfg["N"], cfg["H"], cfg["D"], cfg["E"], torch.bfloat16, seed)
        tokens = cfg["B"] * cfg["N"]
        alg_bytes = tokens * cfg["H"] * (W.BYTES_LAVD_FWD + W.BYTES_LAVD_BWD)
        flops = tokens * cfg["H"] * (W.FLOP_FWD + W.FLOP_BWD)
    elif name == "C5":
        if shape:
            cfg.update(N=int(shape.split(",")[1]), H=int(shape.split(",")[2]))
        from xopes_b200.lightning_attn.seq_parallel import token_range
        rng = token_range(cfg["N"], rank, world)
        w = W.varlen_inputs(cfg["N"], cfg["docs"], cfg["H"], cfg["D"], cfg["E"], torch.bfloat16, 0,
                            token_range=rng, device=dev)
        tokens = cfg["N"]  # the whole stream: ranks split it (strong scaling)
        alg_bytes = tokens * cfg["H"] * W.BYTES_LASD_FWD
        flops = tokens * cfg["H"] * W.FLOP_FWD
    elif base_name(name) == "C4":
        vector = name == "C4v"
        cfg["decay"] = "vector ldk = logsigmoid(N(0,1))/16" if vector else "scalar per head"
        w = W.decode_inputs(cfg["B"], cfg["H"], cfg["D"], cfg["E"], cfg["steps"], vector, seed=seed)
        tokens = cfg["B"] * cfg["steps"]
        alg_bytes = cfg["steps"] * W.decode_bytes_per_step(cfg["B"], cfg["H"], cfg["D"], cfg["E"], vector)
    else:
        raise SystemExit(f"unknown workload {name}")
    return cfg, w, tokens, alg_bytes, flops


def pin(t):
    return t.contiguous().pin_memory()


class LasdStep:
    """Configuration 2: forward + backward of lasd through the public API."""
    launches_per_step = 3  # o pass, dq pass, one launch for the dk and dv passes together
    main_launches = 3      # launches of the dominant kernel among them
    kernel = "chunk_pass_kernel"

    def __init__(self, w, dev):
        import xopes_b200 as xb
        self.xb = xb
        self.dev = dev
        self.host = {k: pin(v) for k, v in w.items()}
        self.d = {k: v.to(dev, non_blocking=True) for k, v in self.host.items()}
        self.h2d = sum(v.numel() * v.element_size() for v in self.host.values())
        self.out_host = None
        # end-to-end leg: inputs double-buffered on the device, copies on their own streams so that
        # the upload of step k+1 and the download of step k overlap the kernels (PCIe is full duplex)
        self.h2d_stream, self.d2h_stream = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.dev_in = [None, None]
        self.in_ev = [torch.cuda.Event(), torch.cuda.Event()]
        self.done_ev = [torch.cuda.Event(), torch.cuda.Event()]
        self.slot = 0
        self.last = None

    def _fb(self, d):
        q, k, v = (d[x].requires_grad_() for x in ("q", "k", "v"))
        o, sf = self.xb.lightning_attn_func(q, k, v, ld=d["ld"], initial_state=d["initial_state"],
                                            decay_type="scalar")
        o.backward(d["do"])
        res = (o.detach(), sf, q.grad, k.grad, v.grad)
        q.grad = k.grad = v.grad = None
        return res

    def step(self):
        self.last = self._fb(self.d)
        return self.last

    def step_e2e(self):
        s = self.slot
        self.slot ^= 1
        main = torch.cuda.current_stream(self.dev)
        if self.dev_in[s] is None:
            self.dev_in[s] = {k: torch.empty(v.shape, dtype=v.dtype, device=self.dev) for k, v in self.host.items()}
            self.done_ev[s].record(main)
        with torch.cuda.stream(self.h2d_stream), torch.no_grad():
            self.h2d_stream.wait_event(self.done_ev[s])  # the step that last used this buffer set is done
            for k, v in self.host.items():
                self.dev_in[s][k].copy_(v, non_blocking=True)
            self.in_ev[s].record(self.h2d_stream)
        main.wait_event(self.in_ev[s])
        res = self._fb(self.dev_in[s])
        self.done_ev[s].record(main)
        if self.out_host is None:
            self.out_host = [torch.empty(r.shape, dtype=r.dtype, pin_memory=True) for r in res]
        with torch.cuda.stream(self.d2h_stream):
            self.d2h_stream.wait_event(self.done_ev[s])
            for hbuf, r in zip(self.out_host, res):
                r.record_stream(self.d2h_stream)
                hbuf.copy_(r, non_blocking=True)
        self.d2h = sum(r.numel() * r.element_size() for r in res)
        return res

    def drain(self):
        """Make the timing stream wait for the copies still in flight (the last download)."""
        torch.cuda.current_stream(self.dev).wait_stream(self.d2h_stream)

    def parity(self):
        """rel-L2 of the last step's outputs against the CPU oracle on two (b,h) pairs."""
        from oracle import lightning_attn_oracle as orc
        o, sf, dq, dk, dv = self.last
        errs = {}
        hh = self.host["q"].shape[2]
        for b, h in ((0, 0), (self.host["q"].shape[0] - 1, hh - 1)):
            sl = lambda t: t[b:b + 1, :, h:h + 1].float()  # noqa: E731
            q, k, v, do = (sl(self.host[x]) for x in ("q", "k", "v", "do"))
            ld = self.host["ld"][h:h + 1]
            s0 = self.host["initial_state"][b:b + 1, h:h + 1]
            ro, rsf = orc.lasd_forward(q, k, v, ld, s0)
            rq, rk, rv, _, _ = orc.lasd_backward(q, k, v, ld, do, s0)
            for n, r, x in (("o", ro, o), ("dq", rq, dq), ("dk", rk, dk), ("dv", rv, dv)):
                errs[n] = max(errs.get(n, 0.0), orc.rel_l2(r, x[b:b + 1, :, h:h + 1].float().cpu()))
            errs["final_state"] = max(errs.get("final_state", 0.0), orc.rel_l2(rsf, sf[b:b + 1, h:h + 1].cpu()))
        return errs


class LavdStep(LasdStep):
    # forward: state-only pass, fold, chunk pass, and two launches that only run if the decay leaves
    # the range of the one before (two-reference chunk pass, scan); backward: 1 state-only pass
    # (reverse flow; the forward-flow states are kept from the forward), 1 fold, 3 chunk passes,
    # 3 + 3 such conditional launches, 1 reverse cumulative sum
    launches_per_step = 17
    main_launches = 4      # o, dq, dk, dv chunk passes
    kernel = "lavd_pass_kernel"

    def _fb(self, d):
        q, k, v, ldk = (d[x].requires_grad_() for x in ("q", "k", "v", "ldk"))
        o, sf = self.xb.lightning_attn_func(q, k, v, ldk=ldk, decay_type="vector")
        o.backward(d["do"])
        res = (o.detach(), sf, q.grad, k.grad, v.grad, ldk.grad)
        q.grad = k.grad = v.grad = ldk.grad = None
        return res

    def parity(self):
        from oracle import lightning_attn_oracle as orc
        o, sf, dq, dk, dv, dldk = self.last
        errs = {}
        hh = self.host["q"].shape[2]
        for b, h in ((0, 0), (self.host["q"].shape[0] - 1, hh - 1)):
            sl = lambda t: t[b:b + 1, :, h:h + 1].float()  # noqa: E731
            q, k, v, do, ldk = (sl(self.host[x]) for x in ("q", "k", "v", "do", "ldk"))
            ro, rsf = orc.lavd_forward(q, k, v, ldk, None)
            rq, rk, rv, rlk, _, _ = orc.lavd_backward(q, k, v, ldk, None, do)
            for n, r, x in (("o", ro, o), ("dq", rq, dq), ("dk", rk, dk), ("dv", rv, dv), ("dldk", rlk, dldk)):
                errs[n] = max(errs.get(n, 0.0), orc.rel_l2(r, x[b:b + 1, :, h:h + 1].float().cpu()))
            errs["final_state"] = max(errs.get("final_state", 0.0), orc.rel_l2(rsf, sf[b:b + 1, h:h + 1].cpu()))
        return errs


class DecodeStep:
    """Configuration 4: one step = the 64-token decode loop, state carried in place."""
    kernel = "decode_kernel"

    def __init__(self, w, dev, vector):
        import xopes_b200 as xb
        self.xb = xb
        self.dev = dev
        self.vector = vector
        self.w = w
        self.ld = w["ld"].to(dev)
        self.state = w["state"].to(dev).clone()
        self.host_toks = [{k: pin(v) for k, v in t.items()} for t in w["steps"]]
        self.toks = [{k: v.to(dev) for k, v in t.items()} for t in self.host_toks]
        self.launches_per_step = self.main_launches = len(self.toks)
        b, _, h, e = self.toks[0]["v"].shape
        self.o = torch.empty(len(self.toks), b, 1, h, e, dtype=torch.bfloat16, device=dev)
        self.h2d = sum(v.numel() * v.element_size() for t in self.host_toks for v in t.values())
        self.out_host = torch.empty(self.o.shape, dtype=self.o.dtype, pin_memory=True)
        self.d2h = self.o.numel() * self.o.element_size()

    def _one(self, i, t):
        if self.vector:
            self.xb.lavd_decode_step(t["q"], t["k"], t["v"], t["ldk"], self.state, out=self.o[i])
        else:
            self.xb.lasd_decode_step(t["q"], t["k"], t["v"], self.ld, self.state, out=self.o[i])

    def step(self):
        for i, t in enumerate(self.toks):
            self._one(i, t)
        return self.o

    def step_e2e(self):
        for i, t in enumerate(self.host_toks):
            self._one(i, {k: v.to(self.dev, non_blocking=True) for k, v in t.items()})
        self.out_host.copy_(self.o, non_blocking=True)
        return self.o

    def parity(self):
        """A fresh 64-step loop from the initial state, against the oracle on the first 4 sequences."""
        from oracle import lightning_attn_oracle as orc
        nb = min(4, self.state.shape[0])
        self.state.copy_(self.w["state"].to(self.dev))
        self.step()
        torch.cuda.synchronize()
        st = self.w["state"][:nb].clone()
        err_o = 0.0
        for i, t in enumerate(self.w["steps"]):
            q, k, v = (t[x][:nb].float() for x in ("q", "k", "v"))
            if self.vector:
                ro, st = orc.decode_step_vector(q, k, v, t["ldk"][:nb], st)
            else:
                ro, st = orc.decode_step_scalar(q, k, v, self.w["ld"], st)
            err_o = max(err_o, orc.rel_l2(ro, self.o[i][:nb].float().cpu()))
        return {"o": err_o, "state": orc.rel_l2(st, self.state[:nb].cpu())}


class VarlenStep:
    """Configuration 5: forward of one packed 1M-token stream of 64 documents.  One GPU runs the
    varlen chunk kernel over the whole stream; with N ranks every rank owns a contiguous token
    range and the ranks exchange chunk-end states (one NCCL all-gather)."""
    kernel = "chunk_pass_kernel"

    def __init__(self, w, dev, world, rank, cfg):
        import xopes_b200 as xb
        self.xb = xb
        self.dev = dev
        self.world, self.rank, self.cfg = world, rank, cfg
        self.d = {k: v for k, v in w.items() if k != "cu_seqlens"}
        self.d["ld"] = self.d["ld"].to(dev)
        self.cu_host = w["cu_seqlens"]
        self.cu = self.cu_host.to(dev)
        # one GPU: per-document weight prefix + chunk pass; a rank: state-only pass, fold of the open
        # document's pieces, fold of the gathered summaries, fold over all pieces, weight prefix,
        # chunk pass (NCCL's own kernel is not counted)
        self.launches_per_step = 2 if world == 1 else 6
        self.main_launches = 1
        self.last = None

    def _fwd(self, d):
        with torch.no_grad():
            if self.world == 1:
                o, st = self.xb.lasd_fn(d["q"], d["k"], d["v"], d["ld"], cu_seqlens=self.cu)
                return o, st, None
            return self.xb.lasd_seqpar_forward(d["q"], d["k"], d["v"], d["ld"], self.cu_host)

    def step(self):
        self.last = self._fwd(self.d)
        return self.last[0]

    def parity(self, heads=(0, 7, 15)):
        """This rank's output on the first 256 tokens after its left boundary and the state of the
        document that straddles that boundary at the end of its local part, against the CPU oracle
        run from that document's first token (which lies on an earlier rank) on three heads."""
        from oracle import lightning_attn_oracle as orc
        from xopes_b200 import workloads as W
        from xopes_b200.lightning_attn.seq_parallel import shard_documents, token_range
        o, states, _ = self.last
        cfg = self.cfg
        cu = [int(x) for x in self.cu_host.tolist()]
        start, end = token_range(cfg["N"], self.rank, self.world)
        plan = shard_documents(cu, start, end)
        doc = plan.doc_ids[0]
        a, b = cu[doc], min(cu[doc + 1], end)
        heads = [h for h in heads if h < cfg["H"]]
        w = W.varlen_inputs(cfg["N"], cfg["docs"], cfg["H"], cfg["D"], cfg["E"], torch.bfloat16, 0,
                            token_range=(a, b), device=self.dev)
        sel = lambda t: t[:, :, heads].float().cpu()  # noqa: E731
        ro, rst = orc.lasd_forward(sel(w["q"]), sel(w["k"]), sel(w["v"]), w["ld"][heads].cpu())
        first_local = max(a, start) - a
        cnt = min(256, b - max(a, start))
        lo = max(a, start) - start
        err_o = orc.rel_l2(ro[:, first_local:first_local + cnt], o[:, lo:lo + cnt, heads].float().cpu())
        err_s = orc.rel_l2(rst[0], states[0][heads].cpu())
        return {"o_first_256_local_tokens": err_o, "straddling_document_state": err_s,
                "document_tokens_before_this_rank": max(0, start - a)}


def quiet_cpu():
    """The parity figures of the previous workload ran the CPU oracle on several threads; their
    worker threads keep spinning for a while after the last parallel region and would compete with
    this process's launch thread (the multi-rank C5 step is a few hundred microseconds of many small
    launches).  One thread from here on, and a pause for the pool to go to sleep."""
    torch.set_num_threads(1)
    time.sleep(0.5)


def time_steps(fn, steps, warmup, world, sampler=None, drain=None):
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if sampler:
        sampler.start()
    ev0 = torch.cuda.Event(enable_timing=True)
    ev1 = torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        fn()
    if drain is not None:
        drain()
    ev1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    if world > 1:
        dist.barrier()
    ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms, clocks


def max_over_ranks(d, world):
    """Element-wise maximum of a dict of floats over the ranks."""
    if world == 1 or d is None:
        return d
    import torch.distributed as dist
    keys = sorted(d)
    t = torch.tensor([float(d[k]) for k in keys], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {k: float(x) for k, x in zip(keys, t.tolist())}


# --------------------------------------------------------------------------------------------
# CPU legs (oracle port of the reference's torch operators)
# --------------------------------------------------------------------------------------------
def _load_workloads():
    """The input generators, without importing anything native."""
    from xopes_b200 import workloads as W
    return W


def cpu_sample(name, cfg, seed=0, pairs=None):
    """Times the CPU oracle on a bounded sample of the workload and scales to the full
    configuration: (b,h) pairs are independent and cost is linear in the sequence length, so the
    full job costs (full pair-tokens / sample pair-tokens) times the sample.  `pairs` bounds the
    number of (b,h) pairs of a C2/C3 sample (None: the default sample, about 10-30 s).  Returns
    (tokens/s for the full configuration, description, threads, seconds spent)."""
    from oracle import lightning_attn_oracle as orc
    W = _load_workloads()
    threads = torch.get_num_threads()
    if name == "C5":
        lens = W.varlen_doc_lengths(cfg["N"], cfg["docs"], 0)
        cu = [0] + [int(x) for x in torch.cumsum(lens, 0)]
        # sample: the shortest document and as many leading documents as fit the token budget
        picks, budget = [int(torch.argmin(lens))], 200000 if pairs is None else pairs * 2048
        for i in range(cfg["docs"]):
            if i not in picks and int(lens[i]) <= budget:
                picks.append(i)
                budget -= int(lens[i])
        ntok, dt = 0, 0.0
        for i in picks:
            w = W.varlen_inputs(cfg["N"], cfg["docs"], cfg["H"], cfg["D"], cfg["E"], torch.bfloat16, 0,
                                token_range=(cu[i], cu[i + 1]))
            t0 = time.perf_counter()
            orc.lasd_forward(w["q"].float(), w["k"].float(), w["v"].float(), w["ld"])
            dt += time.perf_counter() - t0
            ntok += cu[i + 1] - cu[i]
        val = ntok / dt
        sample = (f"oracle lasd forward on {len(picks)} of {cfg['docs']} documents ({ntok} tokens), "
                  f"{dt:.1f} s; documents are independent, cost is linear in tokens")
        return val, sample, threads, dt
    if name == "C2":
        hs = cfg["H"]
        bs = cfg["B"] if pairs is None else max(1, min(cfg["B"], pairs // hs))
        if pairs is not None and pairs < hs:
            hs = max(1, pairs)
        n = cfg["N"]
        w = W.lasd_inputs(bs, n, hs, cfg["D"], cfg["E"], torch.bfloat16, seed)
        f = {k: v.float() for k, v in w.items()}
        t0 = time.perf_counter()
        orc.lasd_forward(f["q"], f["k"], f["v"], f["ld"], f["initial_state"])
        orc.lasd_backward(f["q"], f["k"], f["v"], f["ld"], f["do"], f["initial_state"], None)
        dt = time.perf_counter() - t0
        scale = cfg["B"] * cfg["H"] / (bs * hs)
        val = cfg["B"] * cfg["N"] / (dt * scale)
        sample = (f"oracle lasd fwd+bwd on a (B={bs},H={hs},N={n}) slice, {dt:.1f} s; scaled by "
                  f"B*H/{bs * hs}={scale:.3g} (independent (b,h) recurrences)")
    elif name == "C3":
        bs, hs = cfg["B"], cfg["H"]
        n = 4096 if pairs is None else max(256, min(cfg["N"], pairs * 4096 // (bs * hs)) // 256 * 256)
        w = W.lavd_inputs(bs, n, hs, cfg["D"], cfg["E"], torch.bfloat16, seed)
        f = {k: v.float() for k, v in w.items()}
        t0 = time.perf_counter()
        orc.lavd_forward(f["q"], f["k"], f["v"], f["ldk"], None)
        orc.lavd_backward(f["q"], f["k"], f["v"], f["ldk"], None, f["do"])
        dt = time.perf_counter() - t0
        scale = cfg["N"] / n
        val = cfg["B"] * cfg["N"] / (dt * scale)
        sample = (f"oracle lavd fwd+bwd on a (B={bs},H={hs},N={n}) slice, {dt:.1f} s; scaled by "
                  f"{scale:.3g} (cost is linear in N)")
    else:  # C4 / C4v
        vector = name == "C4v"
        steps = cfg["steps"] if pairs is None else max(1, min(cfg["steps"], pairs // 128))
        w = W.decode_inputs(cfg["B"], cfg["H"], cfg["D"], cfg["E"], steps, vector, seed=seed)
        st = w["state"]
        t0 = time.perf_counter()
        for t in w["steps"]:
            if vector:
                _, st = orc.decode_step_vector(t["q"].float(), t["k"].float(), t["v"].float(), t["ldk"], st)
            else:
                _, st = orc.decode_step_scalar(t["q"].float(), t["k"].float(), t["v"].float(), w["ld"], st)
        dt = time.perf_counter() - t0
        val = cfg["B"] * steps / dt
        sample = f"oracle decode, {steps} of {cfg['steps']} steps at full batch, {dt:.1f} s"
    return val, sample, threads, dt


def run_reference(args, rank, world):
    """Reference arm: the reference's CPU algorithm for the path (oracle port; the reference is
    Python + Triton and its checkout is not present on the GPU box) on the host cores, all of
    them, on the same configuration.  Every step is a bounded sample sized from a calibration run
    so that warm-up + timed steps end within about three minutes; the step count is the one asked
    for."""
    if rank != 0:
        return
    W = _load_workloads()
    name = args.workload
    cfg = dict(W.CONFIGS[base_name(name)])
    torch.set_num_threads(os.cpu_count() or 1)
    total = args.warmup + args.steps
    # calibration: a small sample, to learn the per-pair cost on this box
    cal_pairs = 16
    _, _, _, dt = cpu_sample(name, cfg, seed=10_000, pairs=cal_pairs)
    per_step_budget = max(1.0, 170.0 / total)
    pairs = int(max(4, min(cfg.get("B", 1) * cfg["H"] * 64, cal_pairs * per_step_budget / max(dt, 1e-3))))
    vals, sample, threads = [], "", 1
    for i in range(total):
        val, sample, threads, _ = cpu_sample(name, cfg, seed=i, pairs=pairs)
        if i >= args.warmup:
            vals.append(val)
    val = sum(vals) / len(vals)
    tokens = cfg.get("B", 1) * (cfg.get("N") or cfg.get("steps"))
    line = {
        "impl": "reference", "metric": metric_name(name), "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": len(vals), "warmup": args.warmup,
        "ms_per_step": tokens / val * 1e3, "higher_is_better": True,
        "scaling": "strong" if name == "C5" else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(name, cfg, world),
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": sample + "; ms_per_step is the full configuration at that rate"},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def metric_name(workload):
    return {"C5": "lasd varlen fwd tokens/s (bf16 N1M 64 docs H16 D128)",
            "C2": "lasd fwd+bwd tokens/s (bf16 N8K H32 D128)",
            "C3": "lavd fwd+bwd tokens/s (bf16 N16K H16 D128)",
            "C4": "decode tokens/s (B256 H32 D128, 64-step loop, scalar decay)",
            "C4v": "decode tokens/s (B256 H32 D128, 64-step loop, vector decay)"}[workload]


def workload_config(name, cfg, world):
    c = {"workload": f"{name}: " + {
        "C5": "lasd forward, one packed stream of 64 documents, sequence-sharded across ranks",
        "C2": "lasd forward+backward, per-head scalar decay, fp32 initial state",
        "C3": "lavd forward+backward, ldk = logsigmoid(x)/16, no initial state",
        "C4": "recurrent decode, scalar decay, 64-step loop, fp32 state in place",
        "C4v": "recurrent decode, vector decay (ldk), 64-step loop, fp32 state in place"}[name]}
    c.update({k: v for k, v in cfg.items() if k != "kind"})
    c["partition"] = (f"contiguous token ranges over {world} GPU(s); one all-gather of chunk-end states"
                      if name == "C5" else
                      f"batch x head, one full batch per GPU, {world} GPU(s), no collective")
    c["l2"] = "inputs per step exceed the 126 MB L2 (no flush needed)"
    return c


# --------------------------------------------------------------------------------------------
# one workload on the GPU(s)
# --------------------------------------------------------------------------------------------
def make_runner(name, cfg, w, dev, world, rank):
    if name == "C5":
        return VarlenStep(w, dev, world, rank, cfg)
    if name == "C2":
        return LasdStep(w, dev)
    if name == "C3":
        return LavdStep(w, dev)
    return DecodeStep(w, dev, vector=(name == "C4v"))


def measure(name, args, rank, world, local, dev, primary):
    """Times one configuration; returns the dict of its figures (on every rank)."""
    steps = args.steps if primary else max(3, min(args.steps, 10))
    warmup = max(args.warmup, 3)
    quiet_cpu()
    cfg, w, tokens, alg_bytes, flops = make_workload(name, rank, world, dev, args.shape if primary else None)
    runner = make_runner(name, cfg, w, dev, world, rank)
    strong = name == "C5"
    torch.cuda.synchronize()
    sampler = ClockSampler(local) if rank == 0 else None
    ms, clocks = time_steps(runner.step, steps, warmup, world, sampler)
    ms_step = ms / steps
    nrep = 1 if strong else world  # C5 splits one stream; the others replicate a batch per rank
    value = tokens * nrep / (ms_step * 1e-3)

    e2e = None
    if primary and not args.no_e2e and hasattr(runner, "step_e2e"):
        n_e = max(4, steps // 2)
        ms_e, _ = time_steps(runner.step_e2e, n_e, 2, world, drain=getattr(runner, "drain", None))
        ms_e /= n_e
        e2e = {"value": tokens * nrep / (ms_e * 1e-3), "unit": "tokens/s",
               "h2d_bytes_per_step": int(runner.h2d), "d2h_bytes_per_step": int(runner.d2h),
               "ms_per_step": ms_e}

    parity = None
    if not args.no_parity and args.shape is None:
        torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))
        parity = max_over_ranks(runner.parity(), world)

    peaks = measured_peaks()
    launches = runner.launches_per_step
    per_rank_bytes = alg_bytes / world if strong else alg_bytes
    per_rank_flops = flops / world if strong else flops
    kern_launches = runner.main_launches
    per_launch_bytes = per_rank_bytes / kern_launches
    per_launch_s = ms_step * 1e-3 / kern_launches
    achieved = per_launch_bytes / per_launch_s / 1e9
    kernel = runner.kernel
    if name == "C2":
        from xopes_b200 import _lib
        if _lib.load().la_lasd_path(cfg["N"], cfg["D"], cfg["E"], _lib.LA_BF16, 0) != 1:
            kernel = "scan_kernel"
    traffic, traffic_src = None, None
    ent = traffic_table().get(f"{kernel}:{base_name(name)}")
    if ent is not None:
        th = cfg["N"] * cfg["H"] * (cfg.get("B", 1) if not strong else 1.0 / world)
        traffic = ent["dram_bytes_per_token_head_per_launch"] * th
        traffic_src = ent["source"]
    roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": achieved / peaks["hbm_gbs"], "traffic": traffic, "traffic_source": traffic_src,
            "peak_source": peaks["source"], "kernel": kernel,
            "algorithmic_bytes_per_launch": per_launch_bytes, "avg_launch_ms": per_launch_s * 1e3}
    if flops:
        tf = per_rank_flops / (ms_step * 1e-3) / 1e12
        roof.update({"tensor_tflops": tf, "tensor_peak_tflops": peaks["bf16_tflops"],
                     "tensor_frac": tf / peaks["bf16_tflops"],
                     "tensor_frac_of_nominal_2250": tf / 2250.0,
                     "flop_accounting": "causal intra-chunk tiles at half, chunk 128"})
    res = {
        "metric": metric_name(name), "value": value, "unit": "tokens/s", "ms_per_step": ms_step,
        "steps": steps, "warmup": warmup, "scaling": "strong" if strong else "weak",
        "config": workload_config(name, cfg, world), "clocks": clocks, "e2e": e2e,
        "gpu_launches": launches * steps, "roofline": roof, "parity_rel_l2_vs_cpu_oracle": parity,
    }
    if base_name(name) == "C4":
        res["hbm_gbs"] = achieved
    del runner, w
    torch.cuda.empty_cache()
    return res, cfg


def measure_lasd_shape(b, n, h, dev, steps, world, seed=0):
    """Forward and forward+backward ms of lasd (bf16, D = E = 128, per-head decay, initial state)
    for one (B, N, H); the maximum over ranks."""
    import xopes_b200 as xb
    from xopes_b200 import workloads as W
    quiet_cpu()
    w = W.lasd_inputs(b, n, h, 128, 128, torch.bfloat16, seed)
    d = {k: v.to(dev) for k, v in w.items()}
    q, k, v = (d[x].requires_grad_() for x in ("q", "k", "v"))

    def fwd():
        with torch.no_grad():
            xb.lasd_fn(q, k, v, d["ld"], initial_state=d["initial_state"])

    def fb():
        o, _ = xb.lasd_fn(q, k, v, d["ld"], initial_state=d["initial_state"])
        o.backward(d["do"])
        q.grad = k.grad = v.grad = None

    ms_f, _ = time_steps(fwd, steps, 3, world)
    ms_fb, _ = time_steps(fb, steps, 3, world)
    del d, w
    torch.cuda.empty_cache()
    return ms_f / steps, ms_fb / steps


def measure_lavd_variants(b, n, h, dev, steps, world, seed=0):
    """fwd+bwd ms of two more vector-decay calls at configuration 3's shape: the decay on the value
    features only (ldv: the tensor-core passes with their roles exchanged) and ldk given in bf16
    (read as 16-bit by the kernels).  Maximum over ranks."""
    import xopes_b200 as xb
    from xopes_b200 import workloads as W
    quiet_cpu()
    w = W.lavd_inputs(b, n, h, 128, 128, torch.bfloat16, seed)
    d = {k: v.to(dev) for k, v in w.items()}
    q, k, v = (d[x].requires_grad_() for x in ("q", "k", "v"))
    out = {}
    for name, kw in (("ldv_only", {"ldv": d["ldk"].clone().requires_grad_()}),
                     ("ldk_bf16", {"ldk": d["ldk"].bfloat16().requires_grad_()})):
        def fb():
            o, _ = xb.lightning_attn_func(q, k, v, decay_type="vector", **kw)
            o.backward(d["do"])
            q.grad = k.grad = v.grad = None
            for t in kw.values():
                t.grad = None
        ms, _ = time_steps(fb, steps, 3, world)
        out[name + "_fwd_bwd_ms"] = ms / steps
    del d, w
    torch.cuda.empty_cache()
    return out


def measure_c5_single_gpu(args, rank, world, dev):
    """The whole configuration-5 stream on rank 0's GPU alone (the other ranks wait), so that a
    multi-GPU line carries the one-GPU time it is compared with."""
    import torch.distributed as dist
    ms_step = None
    quiet_cpu()
    if rank == 0:
        steps = max(3, min(args.steps, 10))
        cfg, w, tokens, _, _ = make_workload("C5", 0, 1, dev)
        runner = VarlenStep(w, dev, 1, 0, cfg)
        ms, _ = time_steps(runner.step, steps, 3, 1)
        ms_step = ms / steps
        del runner, w
        torch.cuda.empty_cache()
    dist.barrier()
    return ms_step


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=["C2", "C3", "C4", "C4v", "C5"],
                    help="time this configuration only (default: C2 as the headline, the rest under `secondary`)")
    ap.add_argument("--no-secondary", action="store_true")
    ap.add_argument("--secondary", default="C3,C4,C4v,C5,rows",
                    help="which of the secondary measurements to take (comma-separated)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--shape", default=None, help="B,N,H override (profiling a smaller case)")
    args = ap.parse_args()
    rank, world, local = dist_env()
    only = args.workload is not None
    if args.workload is None:
        args.workload = "C2"
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    res, cfg = measure(args.workload, args, rank, world, local, dev, primary=True)
    secondary = {}
    if not only and not args.no_secondary and args.shape is None:
        want = [x for x in args.secondary.split(",") if x]
        for name in ("C3", "C4", "C4v", "C5"):
            if name not in want:
                continue
            r, _ = measure(name, args, rank, world, local, dev, primary=False)
            r.pop("e2e", None)
            secondary[name] = r
        steps2 = max(3, min(args.steps, 10))
        # the reference's few-pair benchmark row (benchmarks/lightning_attention/README.md:112,123:
        # lasd_p B1 H16 D128 N32768, 1.222 ms forward / 4.174 ms backward on A100): few (sequence,
        # head) pairs, served by the segmented passes
        f, fb = measure_lasd_shape(1, 32768, 16, dev, steps2, world) if "rows" in want else (None, None)
        if f is not None:
            secondary["lasd_B1_N32768_H16"] = {
                "fwd_ms": f, "bwd_ms": fb - f, "fwd_bwd_ms": fb,
                "reference_published_A100_ms": {"fwd": 1.2220, "bwd": 4.1736,
                                                "source": "benchmarks/lightning_attention/README.md:112,123"}}
        if "rows" in want:
            secondary["lavd_variants_B4_N16384_H16"] = measure_lavd_variants(4, 16384, 16, dev, steps2, world)
        # configuration 2 partitioned by batch x head over the ranks (strong scaling): every rank
        # takes B / N of the batches of the same global problem
        if cfg["B"] % world == 0 and "rows" in want:
            f, fb = measure_lasd_shape(cfg["B"] // world, cfg["N"], cfg["H"], dev, steps2, world, seed=rank)
            secondary["C2_strong"] = {
                "scaling": "strong", "batches_per_rank": cfg["B"] // world, "fwd_bwd_ms": fb,
                "value": cfg["B"] * cfg["N"] / (fb * 1e-3), "unit": "tokens/s",
                # the headline step is one full batch on one GPU (every rank runs one), so this is
                # the strong-scaling speed-up of the same global problem
                "speedup_over_full_batch_on_one_gpu": res["ms_per_step"] / fb}
        if world > 1 and "C5" in secondary:
            one = measure_c5_single_gpu(args, rank, world, dev)
            if rank == 0:
                secondary["C5"]["single_gpu_ms_per_step_same_job"] = one
                secondary["C5"]["speedup_over_single_gpu"] = one / secondary["C5"]["ms_per_step"]
    elif args.workload == "C5" and world > 1:
        one = measure_c5_single_gpu(args, rank, world, dev)
        if rank == 0:
            res["single_gpu_ms_per_step_same_job"] = one
            res["speedup_over_single_gpu"] = one / res["ms_per_step"]

    if rank == 0:
        line = {
            "metric": res["metric"], "value": res["value"], "unit": "tokens/s", "n_gpus": world,
            "steps": res["steps"], "warmup": res["warmup"], "ms_per_step": res["ms_per_step"],
            "higher_is_better": True, "scaling": res["scaling"], "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": res["config"], "clocks": res["clocks"],
            "e2e": res["e2e"], "gpu_launches": res["gpu_launches"], "roofline": res["roofline"],
            "parity_rel_l2_vs_cpu_oracle": res["parity_rel_l2_vs_cpu_oracle"],
        }
        for k in ("hbm_gbs", "single_gpu_ms_per_step_same_job", "speedup_over_single_gpu"):
            if k in res:
                line[k] = res[k]
        if secondary:
            line["secondary"] = secondary
        if world == 1 and not args.no_cpu_baseline:
            torch.set_num_threads(os.cpu_count() or 1)
            val, sample, threads, _ = cpu_sample(args.workload, cfg)
            line["cpu_baseline"] = {"value": val, "unit": "tokens/s", "cores": threads,
                                    "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
