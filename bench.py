"""Attention-path benchmark: chunked causal GQA prefill (headline) and q8_0 decode.

python bench.py --gpus N --steps K --warmup W            this library on N B200s
python bench.py --impl reference --gpus N ...            the reference's CPU attention
                                                         (oracle port) on the host cores

Workload (the 8K-context prefill of the reference's bench grid): T=8192 tokens in 2048-token chunks against
the growing q8_0 cache, 24 query / 4 KV heads, head_dim 256, 16 layers with independent
seeds. One step = all 16 layers: per chunk kv_encode_bulk (quantise + append), stage the new
rows, tensor-core chunk attention. `value` = tokens/s with Q/K/V resident in HBM; `e2e` =
the same through the C ABI with pinned HOST buffers (H2D of Q/K/V and D2H of the output
inside the timed region). The same JSON line carries the decode results (depths 672 / 8192 /
32768 / 100000, 128 steps x 16 layers, KV GB/s against the measured HBM peak).

Inputs are seeded synthetic N(0,1) tensors of the named shapes, generated on the device
(torch.randn with per-layer seeds chained from the config's seed the way the reference
chains its layer seeds, crates/hipml-model/src/gpu.rs:814-819).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

H, KV, D, LAYERS = 24, 4, 256, 16
W, QW = KV * D, H * D
ROW = 272
SCALE = 0.0625
T_PREFILL, CHUNK = 8192, 2048
DECODE_DEPTHS = (672, 8192, 32768, 100000)
DECODE_STEPS = 128


def layer_seeds(seed: int, n: int):
    out, s = [], seed
    for _ in range(n):
        out.append(s & 0x7FFF_FFFF_FFFF_FFFF)
        s = (s * 6364136223846793005 + 1) & 0xFFFF_FFFF_FFFF_FFFF
    return out


def chunk_pairs(pos0: int, tokens: int) -> int:
    """Causal (query, key) pairs of one chunk: row t sees pos0 + t + 1 keys."""
    return tokens * pos0 + tokens * (tokens + 1) // 2


def attn_flops(pairs: int) -> float:
    """The reference's own count: 4 * head_dim * n_heads per (query, key) pair
    (crates/hipml-cli/src/attn_chunk_bench.rs:104-106)."""
    return 4.0 * D * H * pairs


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], tflops=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    tflops_burst=p["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, tflops=1400.0, tflops_burst=1590.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index
        self.first = threading.Event()
        self.skip = 0

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms",
                 "50", "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            # the tool takes a moment to start: wait for its first line, and count only the
            # lines that arrive after this point (while the work of the block is running)
            self.first.wait(timeout=5.0)
            self.skip = len(self.rows)
            self.t0 = time.monotonic()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])
            self.first.set()

    def hold(self, fn, seconds=0.6):
        """Keeps the same work running (untimed) until the block has lasted `seconds`, so that
        a short timed region still leaves several samples taken under its load."""
        while self.proc and time.monotonic() - self.t0 < seconds:
            fn()

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows[self.skip:]:
            try:
                sm.append(float(r[1]))
                mx = max(mx, float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm),
                "window": "every 50 ms while the warm-up and timed steps run, and the same step "
                          "repeated (untimed) until the window is 0.6 s long"}


# ------------------------------------------------------------------------------- GPU arm

class Prefill:
    """Device-resident inputs and per-layer caches for the chunked prefill workload."""

    def __init__(self, torch, api, heads, n_kv, tokens, chunk, layers, seed, stride):
        self.torch, self.api = torch, api
        self.heads, self.n_kv, self.tokens, self.chunk, self.layers = heads, n_kv, tokens, chunk, layers
        self.stride = stride
        self.qw, self.w = heads * D, n_kv * D
        dev = "cuda"
        self.q, self.k, self.v = [], [], []
        for s in layer_seeds(seed, layers):
            g = torch.Generator(device=dev).manual_seed(s)
            self.q.append(torch.randn(tokens, self.qw, device=dev, generator=g))
            self.k.append(torch.randn(tokens, self.w, device=dev, generator=g))
            self.v.append(torch.randn(tokens, self.w, device=dev, generator=g))
        self.kc = [torch.zeros(n_kv * stride * ROW, dtype=torch.uint8, device=dev) for _ in range(layers)]
        self.vc = [torch.zeros(n_kv * stride * ROW, dtype=torch.uint8, device=dev) for _ in range(layers)]
        self.out = torch.empty(tokens, self.qw, device=dev)
        self.cap = (tokens + 127) // 128 * 128
        self.ws = torch.empty(api.attn_chunk_workspace_bytes(n_kv, D, 0, self.cap), dtype=torch.uint8,
                              device=dev)
        self.chunks = [(p, min(chunk, tokens - p)) for p in range(0, tokens, chunk)]
        self.launches_per_step = layers * len(self.chunks) * 3
        self.events = None
        self.splits, self.pa, self.pm = 1, None, None
        self.q_parts = None

    def use_key_splits(self, splits, max_rows):
        """Cut every query tile's key range into `splits` slices (partials + combine pass): a
        rank that owns few KV heads has fewer query-tile pairs than the device has SM pairs."""
        self.splits = splits
        self.splits_by_chunk = None      # optional: slices per chunk position (<= splits)
        if splits >= 2:
            qslots = (max_rows + 31) // 32 * 32
            self.pa = self.torch.empty(splits * qslots * self.qw, device="cuda")
            self.pm = self.torch.empty(splits * qslots * self.heads * 2, device="cuda")
        self.count_launches()

    def count_launches(self):
        """Launches of one step: append + staging for every chunk, the attention (and the
        combine pass with key slices) for the chunks this rank attends."""
        n = 0
        for ci in range(len(self.chunks)):
            if self.q_parts is None or self.q_parts[ci][1] > 0:
                n += 2 if self.splits_of(ci) >= 2 else 1
        self.launches_per_step = self.layers * (2 * len(self.chunks) + n)

    def splits_of(self, ci):
        return self.splits if self.splits_by_chunk is None else self.splits_by_chunk[ci]

    def prepare(self, l, ci, ws, k=None, v=None):
        """Append chunk ci of layer l to the q8_0 cache and stage the new rows."""
        pos0, n = self.chunks[ci]
        if k is None:
            k, v = self.k[l], self.v[l]
        self.api.kv_encode_bulk(k[pos0:pos0 + n], v[pos0:pos0 + n], self.kc[l], self.vc[l], self.n_kv,
                                D, self.stride, pos0, 0, n)
        self.api.attn_chunk_stage(self.kc[l], self.vc[l], self.n_kv, D, 1, self.stride, pos0, pos0 + n,
                                  self.cap, ws)

    def attend(self, l, ci, ws, out=None, mode=0, q=None):
        """Chunk attention of this rank's query rows of chunk ci (all rows unless q_parts is set)."""
        pos0, n = self.chunks[ci]
        off, rows = (0, n) if self.q_parts is None else self.q_parts[ci]
        if rows <= 0:
            return
        q = self.q[l] if q is None else q
        out = self.out if out is None else out
        self.api.attn_chunk_staged(q[pos0 + off:pos0 + off + rows], out[pos0 + off:pos0 + off + rows],
                                   self.heads, self.n_kv, D, pos0 + off, rows, self.cap, ws, self.pa,
                                   self.pm, self.splits_of(ci), mode=mode)

    def layer(self, l, ws, mode=0, timed=None, out=None, q=None, k=None, v=None):
        for ci in range(len(self.chunks)):
            self.prepare(l, ci, ws, k, v)
            if timed is not None:
                timed[0][l][ci].record()
            self.attend(l, ci, ws, out, mode, q)
            if timed is not None:
                timed[1][l][ci].record()

    def step(self, mode=0, timed=None):
        """Layer-major: all chunks of a layer, then the next layer, one launch after the other,
        with the staged operand image kept across the chunks of a layer (only the new rows are
        staged). (Running the append + staging of the next chunk on a second stream beside the
        attention was measured: no gain, 34.74 against 34.72 ms per step.)"""
        for l in range(self.layers):
            self.layer(l, self.ws, mode, timed)

    def step_chunk_major(self, mode=0):
        """The reference engine's loop order (crates/hipml-model/src/gpu/prefill.rs:269-285): every
        chunk goes through all layers before the next chunk, through the drop-in entry
        hipml_attn_chunk with ONE workspace, so every call restages all visible keys."""
        for ci, (pos0, n) in enumerate(self.chunks):
            off, rows = (0, n) if self.q_parts is None else self.q_parts[ci]
            for l in range(self.layers):
                self.api.kv_encode_bulk(self.k[l][pos0:pos0 + n], self.v[l][pos0:pos0 + n], self.kc[l],
                                        self.vc[l], self.n_kv, D, self.stride, pos0, 0, n)
                if rows <= 0:
                    continue
                self.api.attn_chunk(self.q[l][pos0 + off:pos0 + off + rows],
                                    self.kc[l], self.vc[l], self.out[pos0 + off:pos0 + off + rows],
                                    self.heads, self.n_kv, D, pos0 + off, rows, 1, self.stride, self.pa,
                                    self.pm, self.splits_of(ci), mode, self.ws)


def run_timed(torch, dist, fn, steps, warmup):
    """W warm-up + K timed steps between CUDA events, barrier + synchronize on both sides;
    returns ms per step as the max over ranks."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    ms = e0.elapsed_time(e1) / steps
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def prefill_e2e(torch, api, L, pf: Prefill, steps, warmup, check=None):
    """The same step through the C ABI with HOST buffers: per layer, Q/K/V go host->device
    from pinned memory and the output comes back, inside the timed region. Three streams
    take the layers in turn, so the host->device engine never waits: with two, the upload of
    layer l + 2 queued behind the download of layer l on the same stream and the engine idled
    about 1 ms per pair of layers (94.8 -> 91.3 ms per step; the upload then runs at 47 GB/s
    beside the download, which is what the link gives in both directions at once)."""
    lib = L.load()
    nbytes_q, nbytes_kv = pf.tokens * pf.qw * 4, pf.tokens * pf.w * 4
    host = []
    for l in range(pf.layers):
        ptrs = []
        for n in (nbytes_q, nbytes_kv, nbytes_kv, nbytes_q):
            p = C.c_void_p()
            L.check("host_alloc", lib.hipml_host_alloc(C.byref(p), n))
            ptrs.append(p)
        host.append(ptrs)
        for src, dst, n in ((pf.q[l], ptrs[0], nbytes_q), (pf.k[l], ptrs[1], nbytes_kv),
                            (pf.v[l], ptrs[2], nbytes_kv)):
            L.check("memcpy", lib.hipml_memcpy(dst, C.c_void_p(src.data_ptr()), n, 2))
    streams = [torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()]
    bufs = []
    for _ in streams:
        bufs.append(dict(q=torch.empty(pf.tokens, pf.qw, device="cuda"),
                         k=torch.empty(pf.tokens, pf.w, device="cuda"),
                         v=torch.empty(pf.tokens, pf.w, device="cuda"),
                         out=torch.empty(pf.tokens, pf.qw, device="cuda"),
                         ws=torch.empty_like(pf.ws)))

    # the query rows this rank attends (all of them, or its share of every chunk) as byte ranges
    row_bytes = pf.qw * 4
    if pf.q_parts is None:
        q_ranges = [(0, nbytes_q)]
    else:
        q_ranges = [((pf.chunks[ci][0] + off) * row_bytes, rows * row_bytes)
                    for ci, (off, rows) in enumerate(pf.q_parts) if rows > 0]

    def step():
        for l in range(pf.layers):
            s, b = streams[l % 3], bufs[l % 3]
            sh = C.c_void_p(s.cuda_stream)
            with torch.cuda.stream(s):
                for at, n in q_ranges:
                    lib.hipml_memcpy_async(C.c_void_p(b["q"].data_ptr() + at), C.c_void_p(host[l][0].value + at),
                                           n, 1, sh)
                lib.hipml_memcpy_async(C.c_void_p(b["k"].data_ptr()), host[l][1], nbytes_kv, 1, sh)
                lib.hipml_memcpy_async(C.c_void_p(b["v"].data_ptr()), host[l][2], nbytes_kv, 1, sh)
                pf.layer(l, b["ws"], out=b["out"], q=b["q"], k=b["k"], v=b["v"])
                for at, n in q_ranges:
                    lib.hipml_memcpy_async(C.c_void_p(host[l][3].value + at), C.c_void_p(b["out"].data_ptr() + at),
                                           n, 2, sh)

    def run():
        main = torch.cuda.current_stream()
        for s in streams:
            s.wait_stream(main)
        step()
        for s in streams:
            main.wait_stream(s)

    ms = run_timed(torch, None, run, steps, warmup)
    parity = None
    if check is not None:
        # layer 0's output rows as they arrived in HOST memory, against the oracle rows
        import numpy as np

        import oracle as O
        idx, want = check
        rows = np.ctypeslib.as_array(C.cast(host[0][3], C.POINTER(C.c_float)), shape=(pf.tokens, pf.qw))
        got = np.array(rows[idx])
        parity = {"rows": int(len(idx)), "max_abs": O.max_abs(want, got), "rel_l2": O.rel_l2(want, got)}
    for ptrs in host:
        for p in ptrs:
            lib.hipml_host_free(p)
    q_bytes = sum(n for _, n in q_ranges)
    h2d = pf.layers * (q_bytes + 2 * nbytes_kv)
    d2h = pf.layers * q_bytes
    return ms, h2d, d2h, parity


def sampled_rows(pf: Prefill, per_chunk=6):
    """Per chunk, `per_chunk` evenly spaced rows inside this rank's share of the chunk's query
    rows (the last row included): [(chunk index, first row, row step, rows in share)]."""
    picks = []
    for ci, (pos0, n) in enumerate(pf.chunks):
        off, rows = (0, n) if pf.q_parts is None else pf.q_parts[ci]
        if rows <= 0:
            continue
        step = max(rows // per_chunk, 1)
        picks.append((ci, (rows - 1) % step, step, off, rows))
    return picks


def prefill_oracle(pf: Prefill, layer=0, per_chunk=6, threads=1):
    """The oracle (CPU port of the reference's attention) on sampled rows of this rank's share
    of layer `layer`, over the dequantised cache the GPU path wrote: the parity reference of
    the timed configuration and the timed CPU baseline in one pass. Returns (global row
    indices, expected rows, timing dict)."""
    import numpy as np

    import oracle as O
    n_keys = pf.tokens
    kb = pf.kc[layer].cpu().numpy().reshape(pf.n_kv, pf.stride, ROW)[:, :n_keys]
    vb = pf.vc[layer].cpu().numpy().reshape(pf.n_kv, pf.stride, ROW)[:, :n_keys]
    kq = O.dequantize_q8(kb).reshape(pf.n_kv, n_keys, D).transpose(1, 0, 2).reshape(n_keys, -1)
    vq = O.dequantize_q8(vb).reshape(pf.n_kv, n_keys, D).transpose(1, 0, 2).reshape(n_keys, -1)
    q = pf.q[layer].cpu().numpy()
    idx, want, dt, pairs = [], [], 0.0, 0
    for ci, r0, step, off, rows in sampled_rows(pf, per_chunk):
        pos0 = pf.chunks[ci][0] + off
        t0 = time.perf_counter()
        w = O.attn_chunk_f32(q[pos0:pos0 + rows], kq, vq, pf.heads, pf.n_kv, D, pos0, rows, SCALE,
                             row0=r0, row_step=step, threads=threads)
        dt += time.perf_counter() - t0
        local = np.arange(r0, rows, step)
        idx.extend((pos0 + local).tolist())
        want.append(w[local])
        pairs += int(sum(pos0 + t + 1 for t in local))
    # seconds per (query, key) pair and head on this host -> one layer of the whole job
    t_layer = dt / (pairs * pf.heads) * chunk_pairs(0, pf.tokens) * H
    return np.array(idx), np.concatenate(want), dict(
        seconds=dt, rows=len(idx), pairs_sample=pairs, tok_s=pf.tokens / (LAYERS * t_layer))


def replay_stats(torch, run, steps, dist=None):
    """Median, min and max ms per step of a replayable `run` of `steps` steps: at least 3
    repetitions and at least 200 ms of device time, at most 20 (the reference's bench rule,
    crates/hipml-cli/src/kvbench.rs:160-163); with `dist`, each repetition is the max over ranks."""
    times = []
    while len(times) < 3 or (sum(times) < 200.0 and len(times) < 20):
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        times.append(ms)
    times.sort()
    return {"median": times[len(times) // 2] / steps, "min": times[0] / steps,
            "max": times[-1] / steps, "reps": len(times)}


def decode_bench(torch, api, depths, steps, layers, hbm_gbs):
    """Single-stream greedy decode: per step and layer ONE launch (hipml_attn_decode_kv_append):
    the split pass quantise-appends the new K/V row, attends over depth+i+1 rows and folds its
    own partials. All steps of one depth are captured
    in one CUDA graph (the reference replays a captured token graph, gpu/graph.rs:43-60), so
    the number is device time, not Python launch time."""
    import numpy as np

    import oracle as O
    results = []
    dev = "cuda"
    for depth in depths:
        stride = depth + steps + 8
        g = torch.Generator(device=dev).manual_seed(2 + depth)
        kc = [torch.zeros(KV * stride * ROW, dtype=torch.uint8, device=dev) for _ in range(layers)]
        vc = [torch.zeros(KV * stride * ROW, dtype=torch.uint8, device=dev) for _ in range(layers)]
        for l in range(layers):
            for p0 in range(0, depth, 8192):
                n = min(8192, depth - p0)
                kf = torch.randn(n, W, device=dev, generator=g)
                vf = torch.randn(n, W, device=dev, generator=g)
                api.kv_encode_bulk(kf, vf, kc[l], vc[l], KV, D, stride, p0, 0, n)
        q = torch.randn(steps, layers, QW, device=dev, generator=g)
        kn = torch.randn(steps, layers, W, device=dev, generator=g)
        vn = torch.randn(steps, layers, W, device=dev, generator=g)
        step_buf = torch.zeros(steps, 8, dtype=torch.int32, device=dev)
        step_buf[:, 0] = torch.arange(depth, depth + steps, dtype=torch.int32, device=dev)
        step_buf[:, 1] = step_buf[:, 0] + 1
        out = torch.empty(steps, layers, QW, device=dev)
        max_splits = 256
        acc = torch.empty(H * max_splits * D, device=dev)
        ml = torch.empty(H * max_splits * 2, device=dev)

        def token(i):
            splits = api.decode_splits(depth + i + 1)
            for l in range(layers):
                api.attn_decode_kv_append(step_buf[i], kn[i, l], vn[i, l], q[i, l], kc[l], vc[l], acc, ml,
                                          out[i, l], H, KV, D, stride, SCALE, splits)

        token(0)  # first-call setup happens outside the capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for i in range(steps):
                    token(i)
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()
        torch.cuda.synchronize()
        stats = replay_stats(torch, graph.replay, steps)
        ms_step = stats["median"]
        # algorithmic bytes: K and V rows of every live position, once per layer
        kv_bytes = sum(layers * 2 * KV * (depth + i + 1) * ROW for i in range(steps)) / steps
        gbs = kv_bytes / (ms_step * 1e-3) / 1e9
        # parity of the timed configuration: last step, layer 0, against the oracle
        i, seq = steps - 1, depth + steps
        kb = kc[0].cpu().numpy().reshape(KV, stride, ROW)
        vb = vc[0].cpu().numpy().reshape(KV, stride, ROW)
        t0 = time.perf_counter()
        want = O.attn_decode_kv_q8(q[i, 0].cpu().numpy(), kb, vb, H, KV, D, seq, SCALE, stride=stride)
        cpu_s = time.perf_counter() - t0
        got = out[i, 0].cpu().numpy()
        results.append({
            "depth": depth, "ms_per_step": ms_step, "ms_per_step_min": stats["min"],
            "ms_per_step_max": stats["max"], "replays": stats["reps"], "tok_s": 1e3 / ms_step,
            "kv_bytes_per_step": kv_bytes, "kv_gbs": gbs, "frac_hbm": gbs / hbm_gbs,
            "l2_assisted": bool(kv_bytes < 126e6 * 3),
            "parity": {"max_abs": O.max_abs(want, got), "rel_l2": O.rel_l2(want, got)},
            "cpu_tok_s_1core": 1.0 / (cpu_s * layers),
            "launches_per_step": layers,
        })
        del kc, vc, graph
        torch.cuda.empty_cache()
    return results


def front_end_bench(torch, api, hbm_gbs, tokens=CHUNK, reps=5):
    """The attention front end of one 2048-token chunk (q|gate split, head RMS norm, M-RoPE,
    q8_0 append): the one-pass fused kernel against the separate launches the reference makes
    (split, norm + rope, kv_encode_bulk), plus the output gate as its own pass. HBM-bound:
    algorithmic bytes per token = q|gate 48 KB in + q 24 KB + gate 24 KB out + k, v 8 KB in +
    2,176 B of cache rows out = 108.7 KB (the separate form re-reads q and k: +56 KB)."""
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(5)
    qg = torch.randn(tokens, H * 2 * D, device=dev, generator=g)
    k = torch.randn(tokens, W, device=dev, generator=g)
    v = torch.randn(tokens, W, device=dev, generator=g)
    qn = 1.0 + 0.1 * torch.randn(D, device=dev, generator=g)
    kn = 1.0 + 0.1 * torch.randn(D, device=dev, generator=g)
    q = torch.empty(tokens, QW, device=dev)
    gate = torch.empty(tokens, QW, device=dev)
    stride = tokens + 8
    kc = torch.zeros(KV * stride * ROW, dtype=torch.uint8, device=dev)
    vc = torch.zeros_like(kc)
    flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=dev)   # larger than L2

    def fused():
        api.attn_front_append_q8(qg, k, v, q, gate, qn, kn, kc, vc, H, KV, D, 64, 1e7, 1e-6, pos0=0,
                                 tokens=tokens, stride=stride)

    k2 = torch.empty_like(k)

    def separate():
        k2.copy_(k)
        api.qg_split_chunk(qg, q, gate, H, D, tokens)
        api.norm_rope_chunk(q, k2, qn, kn, H, KV, D, 64, 1e7, 1e-6, 0, tokens)
        api.kv_encode_bulk(k2, v, kc, vc, KV, D, stride, 0, 0, tokens)

    def gate_pass():
        api.q_gate(q, gate, q, tokens * QW)

    def append_only():
        # the q8_0 quantise + append of the chunk's K/V rows on its own (kv_encode_bulk)
        api.kv_encode_bulk(k, v, kc, vc, KV, D, stride, 0, 0, tokens)

    def timed(fn):
        best = float("inf")
        for _ in range(reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return best

    fused()
    want_k = kc.clone()
    separate()
    same = bool(torch.equal(want_k, kc))
    ms_fused, ms_sep, ms_gate = timed(fused), timed(separate), timed(gate_pass)
    ms_append = timed(append_only)
    bytes_fused = tokens * (H * 2 * D * 4 + 2 * QW * 4 + 2 * W * 4 + 2 * KV * ROW)
    bytes_gate = tokens * QW * 4 * 3
    bytes_append = tokens * (2 * W * 4 + 2 * KV * ROW)      # 8,192 B read + 2,176 B written per token
    return {"tokens": tokens, "fused_ms": ms_fused, "separate_launches_ms": ms_sep,
            "kv_append_bulk_ms": ms_append, "kv_append_bulk_gbs": bytes_append / ms_append / 1e6,
            "kv_append_bulk_frac_hbm": bytes_append / ms_append / 1e6 / hbm_gbs,
            "fused_gbs": bytes_fused / ms_fused / 1e6, "frac_hbm": bytes_fused / ms_fused / 1e6 / hbm_gbs,
            "gate_pass_ms": ms_gate, "gate_pass_gbs": bytes_gate / ms_gate / 1e6,
            "cache_rows_match_separate_form": same,
            "l2": "a 192 MB buffer is rewritten between repetitions"}


def decode_batched(torch, api, slots_list, layers, hbm_gbs, steps=32):
    """Multi-slot decode, B = 8 and 16, per-slot depth uniform in [512, 8192] from seed 3, one
    q8_0 region per slot in a contiguous cache (stride 8448). One step = per layer ONE launch of
    hipml_attn_decode_batch_append (the slots' appends and the fold inside the split pass);
    `steps` steps are captured
    in one CUDA graph. Every slot of the last step is checked against the oracle on layer 0."""
    import numpy as np

    import oracle as O
    dev, stride = "cuda", 8448
    results = []
    for slots in slots_list:
        rng = O.Rng(3)
        depths = [512 + int(rng.uniform() * 7681) for _ in range(slots)]
        g = torch.Generator(device=dev).manual_seed(3 + slots)
        slot_bytes = KV * stride * ROW
        kc = [torch.zeros(slots * slot_bytes, dtype=torch.uint8, device=dev) for _ in range(layers)]
        vc = [torch.zeros(slots * slot_bytes, dtype=torch.uint8, device=dev) for _ in range(layers)]
        for l in range(layers):
            for s, d in enumerate(depths):
                kf = torch.randn(d, W, device=dev, generator=g)
                vf = torch.randn(d, W, device=dev, generator=g)
                api.kv_encode_bulk(kf, vf, kc[l][s * slot_bytes:], vc[l][s * slot_bytes:], KV, D, stride,
                                   0, 0, d)
        splits = api.batch_splits(stride, slots)
        acc_slot, ml_slot = H * splits * D, H * splits * 2
        acc = torch.empty(slots * acc_slot, device=dev)
        ml = torch.empty(slots * ml_slot, device=dev)
        q = torch.randn(steps, layers, slots, QW, device=dev, generator=g)
        kn = torch.randn(steps, layers, slots, W, device=dev, generator=g)
        vn = torch.randn(steps, layers, slots, W, device=dev, generator=g)
        out = torch.empty(steps, layers, slots, QW, device=dev)
        pos = torch.tensor([[[d + i, d + i + 1] for d in depths] for i in range(steps)],
                           dtype=torch.int32, device=dev)

        def token(i):
            for l in range(layers):
                api.attn_decode_batch_append(pos[i], kn[i, l], vn[i, l], q[i, l], kc[l], vc[l], acc, ml,
                                             out[i, l], H, KV, D, stride, SCALE, splits, slot_bytes,
                                             acc_slot, ml_slot, QW, slots)

        token(0)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for i in range(steps):
                    token(i)
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()
        torch.cuda.synchronize()
        stats = replay_stats(torch, graph.replay, steps)
        ms_step = stats["median"]
        kv_bytes = sum(layers * 2 * KV * (d + i + 1) * ROW for d in depths for i in range(steps)) / steps
        gbs = kv_bytes / (ms_step * 1e-3) / 1e9
        worst_abs, worst_rel, i = 0.0, 0.0, steps - 1
        kb = kc[0].cpu().numpy().reshape(slots, KV, stride, ROW)
        vb = vc[0].cpu().numpy().reshape(slots, KV, stride, ROW)
        for s, d in enumerate(depths):
            want = O.attn_decode_kv_q8(q[i, 0, s].cpu().numpy(), kb[s], vb[s], H, KV, D, d + steps, SCALE,
                                       stride=stride)
            got = out[i, 0, s].cpu().numpy()
            worst_abs = max(worst_abs, O.max_abs(want, got))
            worst_rel = max(worst_rel, O.rel_l2(want, got))
        results.append({"slots": slots, "depths": depths, "splits": splits, "ms_per_step": ms_step,
                        "ms_per_step_min": stats["min"], "ms_per_step_max": stats["max"],
                        "replays": stats["reps"], "launches_per_step": layers,
                        "tok_s": slots * 1e3 / ms_step, "kv_bytes_per_step": kv_bytes, "kv_gbs": gbs,
                        "frac_hbm": gbs / hbm_gbs, "l2_assisted": True,
                        "parity": {"max_abs": worst_abs, "rel_l2": worst_rel}})
        del kc, vc, graph
        torch.cuda.empty_cache()
    return results


def prefill_long(torch, api, tokens, heads, n_kv, q_part=None, layers=1, reps=2, key_splits=1,
                 kv_seed=4, slices_at=None):
    """A `tokens`-token causal prefill in 2048-token chunks over the q8_0 cache (stride
    tokens + 8), timed per layer. The same Q/K/V serve every repetition; (heads, n_kv) are this
    rank's shard; q_part(ci, n) -> (offset, rows) selects the rank's share of a chunk's query
    rows (None = all). Returns (ms per layer, parity): sampled rows of the first, the middle and
    the last chunk of this rank's share against the oracle over the dequantised cache."""
    import numpy as np

    import oracle as O
    dev = "cuda"
    stride = tokens + 8
    qw, w = heads * D, n_kv * D
    g = torch.Generator(device=dev).manual_seed(kv_seed)
    q = torch.randn(tokens, qw, device=dev, generator=g)
    k = torch.randn(tokens, w, device=dev, generator=g)
    v = torch.randn(tokens, w, device=dev, generator=g)
    out = torch.full((tokens, qw), float("nan"), device=dev)
    kc = torch.zeros(n_kv * stride * ROW, dtype=torch.uint8, device=dev)
    vc = torch.zeros_like(kc)
    cap = (tokens + 127) // 128 * 128
    ws = torch.empty(api.attn_chunk_workspace_bytes(n_kv, D, 0, cap), dtype=torch.uint8, device=dev)
    chunks = [(p, min(CHUNK, tokens - p)) for p in range(0, tokens, CHUNK)]
    pa = pm = None
    if key_splits >= 2:   # a rank with few query-tile pairs cuts every tile's key range
        qslots = (CHUNK + 31) // 32 * 32
        pa = torch.empty(key_splits * qslots * qw, device=dev)
        pm = torch.empty(key_splits * qslots * heads * 2, device=dev)

    # (the policy is evaluated once, outside the timed loop: it is host arithmetic)
    slices = [key_splits if slices_at is None else min(key_splits, slices_at(p)) for p, _ in chunks]
    parts = [(0, n) if q_part is None else q_part(ci, n) for ci, (_, n) in enumerate(chunks)]

    def layer():
        for ci, (pos0, n) in enumerate(chunks):
            api.kv_encode_bulk(k[pos0:pos0 + n], v[pos0:pos0 + n], kc, vc, n_kv, D, stride, pos0, 0, n)
            api.attn_chunk_stage(kc, vc, n_kv, D, 1, stride, pos0, pos0 + n, cap, ws)
            off, rows = parts[ci]
            if rows > 0:
                api.attn_chunk_staged(q[pos0 + off:pos0 + off + rows], out[pos0 + off:pos0 + off + rows],
                                      heads, n_kv, D, pos0 + off, rows, cap, ws, pa, pm, slices[ci])

    layer()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(layers):
            layer()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / layers)
    assert api.check_device_status() == 0
    # parity: 3 rows each of the first, middle and last chunk (the last row of each included)
    kb = kc.cpu().numpy().reshape(n_kv, stride, ROW)[:, :tokens]
    vb = vc.cpu().numpy().reshape(n_kv, stride, ROW)[:, :tokens]
    kq = O.dequantize_q8(kb).reshape(n_kv, tokens, D).transpose(1, 0, 2).reshape(tokens, -1)
    del kb
    vq = O.dequantize_q8(vb).reshape(n_kv, tokens, D).transpose(1, 0, 2).reshape(tokens, -1)
    del vb
    worst_abs = worst_rel = 0.0
    checked = []
    for ci in sorted({0, len(chunks) // 2, len(chunks) - 1}):
        pos0, n = chunks[ci]
        off, rows = (0, n) if q_part is None else q_part(ci, n)
        if rows <= 0:
            continue
        step = max(rows // 3, 1)
        r0 = (rows - 1) % step
        local = np.arange(r0, rows, step)
        qs = q[pos0 + off:pos0 + off + rows].cpu().numpy()
        want = O.attn_chunk_f32(qs, kq, vq, heads, n_kv, D, pos0 + off, rows, SCALE, row0=r0,
                                row_step=step, threads=min(os.cpu_count() or 1, 16))[local]
        got = out[pos0 + off:pos0 + off + rows].cpu().numpy()[local]
        worst_abs = max(worst_abs, O.max_abs(want, got))
        worst_rel = max(worst_rel, O.rel_l2(want, got))
        checked.append([int(pos0 + off), int(len(local))])
    finite = bool(torch.isfinite(out if q_part is None else out[~torch.isnan(out[:, 0])]).all().item())
    return min(times), {"max_abs": worst_abs, "rel_l2": worst_rel, "chunks_pos0_rows": checked,
                        "finite": finite}


def decode_sharded(torch, dist, api, depth, steps, layers, world, rank, hbm_gbs):
    """Decode at `depth` with the cache rows split across the ranks by sequence. Two forms:
    (a) per layer the owner of the new position appends its row inside the split pass, every
    rank folds its rows to one (acc, max, sum) triple per head (one launch), the triples are
    all-gathered over NCCL and folded again on every rank; (b) ONE launch per layer: the split
    pass appends, folds, stores its triples into every rank's table over NVLink, waits for the
    peers' and writes the output. One CUDA graph per rank holds all steps. The last step of
    layer 0 of either form is checked on rank 0 against the oracle over the gathered cache."""
    import numpy as np

    import oracle as O
    from hipml_b200 import sharding
    dev = "cuda"
    capacity = depth + steps + 8
    lo, hi = sharding.decode_shard_range(capacity, world, rank)
    stride = max(hi - lo, 1)
    g = torch.Generator(device=dev).manual_seed(4 + 17 * rank)
    kc = [torch.zeros(KV * stride * ROW, dtype=torch.uint8, device=dev) for _ in range(layers)]
    vc = [torch.zeros(KV * stride * ROW, dtype=torch.uint8, device=dev) for _ in range(layers)]
    n0 = sharding.local_length(depth, lo, hi)
    for l in range(layers):
        for p0 in range(0, n0, 8192):
            n = min(8192, n0 - p0)
            api.kv_encode_bulk(torch.randn(n, W, device=dev, generator=g),
                               torch.randn(n, W, device=dev, generator=g), kc[l], vc[l], KV, D,
                               stride, p0, 0, n)
    gs = torch.Generator(device=dev).manual_seed(4)  # same query / new rows on every rank
    q = torch.randn(steps, layers, QW, device=dev, generator=gs)
    kn = torch.randn(steps, layers, W, device=dev, generator=gs)
    vn = torch.randn(steps, layers, W, device=dev, generator=gs)
    step_host = []
    for i in range(steps):
        pos = depth + i
        step_host.append([max(pos - lo, 0), sharding.local_length(pos + 1, lo, hi), 0, 0, 0, 0, 0, 0])
    step_buf = torch.tensor(step_host, dtype=torch.int32, device=dev)
    owners = [sharding.decode_owner(depth + i, capacity, world) for i in range(steps)]
    out = torch.empty(steps, layers, QW, device=dev)
    acc = torch.empty(H * 256 * D, device=dev)
    ml = torch.empty(H * 256 * 2, device=dev)
    shard = torch.empty(H, D + 2, device=dev)
    gathered = torch.empty(world, H, D + 2, device=dev)

    def token_nccl(i):
        splits = api.decode_splits(max(step_host[i][1], 1))
        for l in range(layers):
            if owners[i] == rank:
                api.kv_encode(step_buf[i], kn[i, l], vn[i, l], kc[l], vc[l], KV, D, stride)
            api.attn_decode_kv_shard(step_buf[i], q[i, l], kc[l], vc[l], acc, ml, shard, H, KV, D,
                                     stride, SCALE, splits)
            dist.all_gather_into_tensor(gathered, shard)
            api.attn_decode_combine(gathered, out[i, l], H, D, world)

    # The exchange inside the kernel: every rank's workspace is mapped by all ranks (torch's
    # symmetric memory; no multicast binding is asked for) and the split pass stores its
    # triples straight into the peers' tables.
    peer_ws, symm_note = None, None
    try:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        nbytes = api.decode_exchange_bytes(H, D, world)
        ws_t = symm_mem.empty(nbytes, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
        hdl = symm_mem.rendezvous(ws_t, dist.group.WORLD)
        ws_t.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        peer_ws = [int(a) for a in hdl.buffer_ptrs]
    except Exception as e:  # no symmetric memory on this box: the NCCL form only
        symm_note = f"{type(e).__name__}: {e}"[:160]

    def token_peer(i):
        splits = api.decode_splits(max(step_host[i][1], 1))
        own = owners[i] == rank
        for l in range(layers):
            api.attn_decode_kv_shard_exchange_append(
                step_buf[i], kn[i, l] if own else None, vn[i, l] if own else None, q[i, l], kc[l], vc[l],
                acc, ml, out[i, l], H, KV, D, stride, SCALE, splits, peer_ws, rank)

    def token_by_head(i):
        # the result divided by head: head h's triples go to rank h / (H / world) alone, which
        # writes that head's output row (what a row-parallel output projection reads): the split
        # pass sends each triple once, so it is one launch per layer at any rank count
        splits = api.decode_splits(max(step_host[i][1], 1))
        own = owners[i] == rank
        for l in range(layers):
            api.attn_decode_kv_shard_exchange_append(
                step_buf[i], kn[i, l] if own else None, vn[i, l] if own else None, q[i, l], kc[l], vc[l],
                acc, ml, out[i, l], H, KV, D, stride, SCALE, splits, peer_ws, rank, phases=7)

    def measure(token):
        token(0)
        torch.cuda.synchronize()
        dist.barrier()
        mode = "cuda graph"
        try:
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    for i in range(steps):
                        token(i)
            torch.cuda.current_stream().wait_stream(side)
            run = graph.replay
        except Exception as e:  # capture refused: time the eager loop instead
            mode = f"eager ({type(e).__name__})"

            def run():
                for i in range(steps):
                    token(i)
        run()
        torch.cuda.synchronize()
        stats = replay_stats(torch, run, steps, dist)
        return stats, mode, out[steps - 1].clone()

    st_nccl, mode_nccl, out_nccl = measure(token_nccl)
    ms_nccl = st_nccl["median"]
    stats, ms_step, mode, exchange = st_nccl, ms_nccl, mode_nccl, "nccl all_gather"
    peer, out_peer = None, None
    if peer_ws is not None:
        out.zero_()
        st_peer, mode_peer, out_peer = measure(token_peer)
        ok = api.check_device_status() == 0
        same = bool(torch.allclose(out_peer, out_nccl, rtol=0, atol=1e-6))
        # up to 2 ranks the split pass publishes and collects itself; beyond that the exchange is
        # a second launch of (head, rank) CTAs (one SM cannot feed NVLink for many peers)
        one_launch = world <= 2
        peer = {"ms_per_step": st_peer["median"], "ms_per_step_min": st_peer["min"],
                "ms_per_step_max": st_peer["max"], "launch": mode_peer, "status_ok": ok,
                "matches_nccl_form": same, "launches_per_step": layers * (1 if one_launch else 2)}
        if ok and same and st_peer["median"] < ms_nccl:
            stats, ms_step, mode = st_peer, st_peer["median"], mode_peer
            exchange = ("peer-memory stores inside the split pass" if one_launch else
                        "peer-memory stores by an exchange launch after the split pass")
    finite = bool(torch.isfinite(out).all().item())     # of the replicated forms' outputs
    by_head, out_by_head = None, None
    if peer_ws is not None and H % world == 0:
        out.fill_(float("nan"))
        st_bh, mode_bh, last = measure(token_by_head)
        ok = api.check_device_status() == 0
        per = H // world
        mine = last[0].view(H, D)[rank * per:(rank + 1) * per].contiguous()
        rest_untouched = bool(torch.isnan(torch.cat([last[0].view(H, D)[:rank * per],
                                                     last[0].view(H, D)[(rank + 1) * per:]])).all().item())
        out_by_head = torch.empty(world, per, D, device=dev)
        dist.all_gather_into_tensor(out_by_head, mine)
        by_head = {"ms_per_step": st_bh["median"], "ms_per_step_min": st_bh["min"],
                   "ms_per_step_max": st_bh["max"], "launch": mode_bh, "status_ok": ok,
                   "launches_per_step": layers, "heads_per_rank": per,
                   "other_rows_untouched": rest_untouched,
                   "note": "every rank holds the output rows of its H / ranks heads only (the input "
                           "layout of a row-parallel output projection); not the replicated "
                           "result the other two forms give, so it is reported beside them"}
    # parity: layer 0's cache shards gathered on rank 0, last step against the oracle
    pad = max(sharding.decode_shard_range(capacity, world, r)[1] -
              sharding.decode_shard_range(capacity, world, r)[0] for r in range(world))
    parity = None
    both = []
    for c in (kc[0], vc[0]):
        mine = torch.zeros(KV, pad, ROW, dtype=torch.uint8, device=dev)
        mine[:, :stride] = c.view(KV, stride, ROW)
        allc = torch.empty(world, KV, pad, ROW, dtype=torch.uint8, device=dev)
        dist.all_gather_into_tensor(allc, mine)
        both.append(allc)
    if rank == 0:
        seq = depth + steps
        whole = []
        for allc in both:
            parts = []
            for r in range(world):
                rlo, rhi = sharding.decode_shard_range(capacity, world, r)
                parts.append(allc[r, :, :rhi - rlo].cpu().numpy())
            whole.append(np.concatenate(parts, axis=1))
        want = O.attn_decode_kv_q8(q[steps - 1, 0].cpu().numpy(), whole[0], whole[1], H, KV, D, seq,
                                   SCALE, stride=capacity)
        parity = {"nccl_form": {"max_abs": O.max_abs(want, out_nccl[0].cpu().numpy()),
                                "rel_l2": O.rel_l2(want, out_nccl[0].cpu().numpy())}}
        if out_peer is not None:
            parity["peer_form"] = {"max_abs": O.max_abs(want, out_peer[0].cpu().numpy()),
                                   "rel_l2": O.rel_l2(want, out_peer[0].cpu().numpy())}
        if out_by_head is not None:
            got = out_by_head.reshape(-1).cpu().numpy()      # rank order = head order
            parity["by_head_form"] = {"max_abs": O.max_abs(want, got), "rel_l2": O.rel_l2(want, got)}
    del both
    kv_bytes = sum(layers * 2 * KV * (depth + i + 1) * ROW for i in range(steps)) / steps
    gbs = kv_bytes / (ms_step * 1e-3) / 1e9
    return {"depth": depth, "ranks": world, "partition": "sequence", "launch": mode,
            "exchange": exchange, "ms_per_step_nccl": ms_nccl, "peer_memory_exchange": peer,
            "peer_memory_exchange_by_head": by_head,
            "symmetric_memory_error": symm_note,
            "ms_per_step": ms_step, "ms_per_step_min": stats["min"], "ms_per_step_max": stats["max"],
            "replays": stats["reps"], "tok_s": 1e3 / ms_step, "kv_bytes_per_step": kv_bytes,
            "kv_gbs": gbs, "frac_hbm_of_all_gpus": gbs / (hbm_gbs * world),
            "exchange_bytes_per_layer_step": world * H * (D + 2) * 4,
            "parity": parity, "finite": finite}


WORKLOAD = "prefill T=8192 in 2048-token chunks, q8_0 KV, 24/4/256, 16 layers (BASELINE configs[1])"
L2_NOTE = "inputs larger than L2 (7.6 GB of Q/K/V per step)"

# dram__bytes_read.sum + dram__bytes_write.sum of one attn_chunk_tc launch on the 2048-row chunk
# at position 6144 (ncu capture summarised in profiles/attn_chunk_tc_2048_at_6144.md), and the
# algorithmic bytes of that launch (Q in, out, the staged K/V image once); other chunks are
# scaled by their algorithmic bytes.
NCU_CHUNK_TRAFFIC_BYTES = 143.0e6
NCU_CHUNK_ALGORITHMIC_BYTES = 2 * CHUNK * QW * 4 + 8192 * 8192


def chunk_algorithmic_bytes(pos0, n, heads=H, n_kv=KV):
    return 2 * n * heads * D * 4 + (pos0 + n) * n_kv * 2048


def gpu_main(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
    import __graft_entry__ as entry
    entry.build()
    import oracle as O
    from hipml_b200 import _lib as L, api
    pk = peaks()
    if args.decode_only and world > 1:
        # (development aid: the sequence-split decode leg alone)
        r = decode_sharded(torch, dist, api, args.depth, DECODE_STEPS, LAYERS, world, rank, pk["hbm_gbs"])
        if rank == 0:
            print(json.dumps(r))
        dist.barrier()
        dist.destroy_process_group()
        return

    def rank_max(x):
        if dist is None:
            return float(x)
        t = torch.tensor([float(x)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # KV-head sharding: each rank owns n_kv/world KV heads and their query heads; no data-path
    # collective inside the attention. Beyond 4 ranks the ranks that share a KV head divide the
    # chunks (or, --query-partition rows, every chunk's query rows) between them.
    from hipml_b200 import sharding
    kv_shards, q_shards, kv_index, q_index, n_kv_local, heads_local = sharding.kv_head_shard(
        H, KV, world, rank)
    pf = Prefill(torch, api, heads_local, n_kv_local, T_PREFILL, CHUNK, LAYERS,
                 seed=1 + 1000 * kv_index, stride=T_PREFILL + 8)
    by_chunks = args.query_partition == "chunks"

    def q_part(ci, n, n_chunks):
        """This rank's query rows of chunk ci among the ranks that share its KV head."""
        if by_chunks:
            return sharding.chunk_part(ci, n_chunks, n, q_shards, q_index)
        return sharding.query_part(ci, n, q_shards, q_index)

    if q_shards > 1:
        pf.q_parts = [q_part(ci, n, len(pf.chunks)) for ci, (p, n) in enumerate(pf.chunks)]
    # key slices per query tile, by chunk position (the cost model of sharding.py: fewer where the
    # query tiles see few key tiles, more where a rank has few tiles or the tiles are very long)
    def slices_at(p0):
        return sharding.prefill_key_splits(CHUNK if by_chunks else CHUNK // q_shards,
                                           heads_local // n_kv_local, n_kv_local, pos0=p0)

    by_chunk_splits = [slices_at(p) for p, n in pf.chunks]
    key_splits = max(by_chunk_splits)
    pf.use_key_splits(key_splits, CHUNK)
    pf.splits_by_chunk = by_chunk_splits
    pf.count_launches()

    gpu_index = local
    with ClockSampler(gpu_index) as clocks:
        ms_layer_major = run_timed(torch, dist, lambda: pf.step(), args.steps, args.warmup)

        def more():
            pf.step()
            torch.cuda.synchronize()
        clocks.hold(more)
    assert api.check_device_status() == 0

    # per-launch timing of the dominant kernel (the tensor-core chunk attention; with key slices
    # the bracket also holds the small combine pass), on every rank, straight after the timed
    # steps (the same power and clock state)
    def kernel_time(mode):
        ev = [[[torch.cuda.Event(enable_timing=True) for _ in pf.chunks] for _ in range(LAYERS)]
              for _ in range(2)]
        pf.step(mode=mode, timed=ev)
        torch.cuda.synchronize()
        per = [[ev[0][l][c].elapsed_time(ev[1][l][c]) for c in range(len(pf.chunks))] for l in range(LAYERS)]
        return per

    per0 = kernel_time(0)
    # the same job in the reference engine's loop order, through the drop-in entry, and the
    # layer-major form again right after it: the two are compared in the same power / clock
    # state (the device slows down over the first seconds of sustained tensor work)
    ms_chunk_major = run_timed(torch, dist, lambda: pf.step_chunk_major(), args.steps, 1)
    ms_layer_major_again = run_timed(torch, dist, lambda: pf.step(), args.steps, 1)
    assert api.check_device_status() == 0
    # headline: the layer-major form, unless the drop-in order is more than 3 % slower
    headline = "layer-major (staged image kept across a layer's chunks)"
    ms = ms_layer_major
    if ms_chunk_major > 1.03 * ms_layer_major_again:
        headline, ms = "chunk-major through hipml_attn_chunk (full restage per call)", ms_chunk_major
    tok_s = T_PREFILL / (ms * 1e-3)
    parallelism = (f"kv_head x{kv_shards}"
                   + (f", query x{q_shards} by {'chunk pairs' if by_chunks else 'rows of every chunk'}"
                      if q_shards > 1 else "")
                   + (f", key slices {pf.splits_by_chunk} by chunk" if key_splits > 1 else ""))

    line = {
        "metric": "attn prefill tok/s", "value": tok_s, "unit": "tok/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16x2 operands, f32 accumulate",
        "data": "synthetic N(0,1), seeded, generated on device",
        "config": {"workload": WORKLOAD, "l2": L2_NOTE},
        "parallelism": parallelism,
        "loop_order": {"headline": headline, "layer_major_ms": ms_layer_major,
                       "chunk_major_ms": ms_chunk_major,
                       "layer_major_ms_right_after_chunk_major": ms_layer_major_again,
                       "chunk_major_tok_s": T_PREFILL / (ms_chunk_major * 1e-3)},
        "gpu_launches": pf.launches_per_step * args.steps,
        "clocks": clocks.summary(),
    }

    def share(c, n):
        """This rank's part of chunk c's query rows (its causal work differs a little between
        the halves of a chunk; the by-chunk rate is indicative)."""
        return 1.0 if pf.q_parts is None else pf.q_parts[c][1] / n

    def roofline_of(per, issued):
        kernel_ms = rank_max(sum(sum(r) for r in per))       # the slowest rank's kernel time
        flops = LAYERS * sum(attn_flops(chunk_pairs(p, n)) for p, n in pf.chunks)   # whole job
        n_launch = LAYERS * len(pf.chunks)
        achieved = flops / (kernel_ms * 1e-3) / 1e12
        alg_bytes = sum(chunk_algorithmic_bytes(p, n) for p, n in pf.chunks) / len(pf.chunks)
        return {
            "bound": "tensor", "kernel": "attn_chunk_tc", "achieved": achieved,
            "peak": pk["tflops"] * world, "unit": "TFLOP/s", "frac": achieved / (pk["tflops"] * world),
            "traffic": NCU_CHUNK_TRAFFIC_BYTES * alg_bytes / NCU_CHUNK_ALGORITHMIC_BYTES,
            "traffic_note": "ncu dram bytes of the 2048@6144 launch scaled by algorithmic bytes "
                            "to the mean launch of the step (whole job, all ranks)",
            "algorithmic_bytes_per_launch": alg_bytes,
            "peak_source": pk["source"] + " (sustained cuBLAS bf16" + (f", x{world} GPUs)" if world > 1 else ")"),
            "launches": n_launch, "avg_launch_ms": kernel_ms / n_launch,
            "algorithmic_flop_per_launch": flops / n_launch,
            "issued_over_algorithmic": issued,
            "kernel_share_of_step": kernel_ms / ms_layer_major,
            # the same per chunk position on this rank (mean over layers): [pos0, ms, TFLOP/s of
            # the rank's share]
            "by_chunk": [[p, sum(per[l][c] for l in range(LAYERS)) / LAYERS,
                          attn_flops(chunk_pairs(p, n)) / kv_shards * share(c, n) * LAYERS /
                          max(sum(per[l][c] for l in range(LAYERS)) * 1e9, 1e-9)]
                         for c, (p, n) in enumerate(pf.chunks)],
        }

    line["roofline"] = roofline_of(per0, 3.0)

    # parity of the timed configuration + CPU baseline (the reference's own loop, one thread),
    # on every rank over its own share; the worst rank is reported
    idx, want, cpu = prefill_oracle(pf, per_chunk=80)   # ~10 s of one host core at N = 1
    pf.out.fill_(float("nan"))
    pf.layer(0, pf.ws)
    torch.cuda.synchronize()
    got = pf.out.cpu().numpy()[idx]
    line["parity"] = {"rows_per_rank": int(len(idx)), "max_abs": rank_max(O.max_abs(want, got)),
                      "rel_l2": rank_max(O.rel_l2(want, got)), "ranks_checked": world}
    line["cpu_baseline"] = {
        "value": cpu["tok_s"], "unit": "tok/s", "cores": 1, "kind": "port",
        "sample": f"{cpu['rows']} rows x {pf.heads} heads of layer 0 spread over the chunks "
                  f"({cpu['seconds']:.1f} s on rank 0), scaled by causal pair count and head count to "
                  "the whole 16-layer job"}
    # the single-pass precision (the reference kernel's own, attn_chunk_wmma.hip:187-399) beside
    # the compensated default: its error against the same oracle rows and its rates
    per1 = kernel_time(1)
    pf.out.fill_(float("nan"))
    pf.layer(0, pf.ws, mode=1)
    torch.cuda.synchronize()
    got1 = pf.out.cpu().numpy()[idx]
    r1 = roofline_of(per1, 1.0)
    ms_mode1 = run_timed(torch, dist, lambda: pf.step(mode=1), 2, 1)
    line["precision_modes"] = {
        "0 (default: hi*hi + lo*hi + hi*lo, meets rel-L2 1e-4)": {
            "max_abs": line["parity"]["max_abs"], "rel_l2": line["parity"]["rel_l2"],
            "algorithmic_tflops": line["roofline"]["achieved"],
            "issued_tflops": 3.0 * line["roofline"]["achieved"], "ms_per_step": ms_layer_major},
        "1 (single f16 pass, the reference kernel's precision; misses rel-L2 1e-4)": {
            "max_abs": rank_max(O.max_abs(want, got1)), "rel_l2": rank_max(O.rel_l2(want, got1)),
            "algorithmic_tflops": r1["achieved"], "issued_tflops": r1["achieved"],
            "frac_of_peak": r1["frac"], "ms_per_step": ms_mode1}}

    e2e_ms, h2d, d2h, e2e_parity = prefill_e2e(torch, api, L, pf, max(args.steps // 2, 1), 1,
                                               check=(idx, want))
    e2e_ms = rank_max(e2e_ms)
    e2e_parity["max_abs"] = rank_max(e2e_parity["max_abs"])
    e2e_parity["rel_l2"] = rank_max(e2e_parity["rel_l2"])
    line["e2e"] = {"value": T_PREFILL / (e2e_ms * 1e-3), "unit": "tok/s",
                   "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d * world,
                   "d2h_bytes_per_step": d2h * world,
                   "parity_of_host_output": e2e_parity,
                   "note": "per rank: the Q rows it attends and its heads' K/V up from pinned host "
                           "memory, its output rows down, inside the timed region; bytes are the "
                           "sum over ranks"}
    if world > 1:
        # What a consumer that needs whole [T][6144] rows (the output projection) would add:
        # an all-gather of every rank's output share of one layer. Not part of the attention
        # step and not in the headline; reported on its own.
        if pf.q_parts is None:
            share = pf.out
        else:
            share = torch.cat([pf.out[p + off:p + off + rows] for (p, n), (off, rows)
                               in zip(pf.chunks, pf.q_parts) if rows > 0]).contiguous()
        sizes = torch.tensor([share.numel()], device="cuda", dtype=torch.int64)
        dist.all_reduce(sizes, op=dist.ReduceOp.MAX)
        if int(sizes.item()) == share.numel():          # equal shares (the partitions here give that)
            gathered = torch.empty(world * share.numel(), device="cuda")
            for _ in range(2):
                dist.all_gather_into_tensor(gathered, share.reshape(-1))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            dist.barrier()
            e0.record()
            for _ in range(5):
                dist.all_gather_into_tensor(gathered, share.reshape(-1))
            e1.record()
            torch.cuda.synchronize()
            ms_gather = rank_max(e0.elapsed_time(e1) / 5)
            line["gather_for_wo"] = {
                "ms_per_layer": ms_gather, "bytes_per_rank": share.numel() * 4,
                "bus_gbs": (world - 1) * share.numel() * 4 / (ms_gather * 1e-3) / 1e9,
                "ms_per_step_16_layers": ms_gather * LAYERS,
                "note": "NCCL all-gather of the ranks' output shares of one layer; outside the "
                        "timed step (the attention itself needs no collective)"}
            del gathered
        del share
    if world == 1 and not args.no_decode:
        del pf
        torch.cuda.empty_cache()
        line["decode"] = decode_bench(torch, api, DECODE_DEPTHS, DECODE_STEPS, LAYERS,
                                      pk["hbm_gbs"])
        line["decode_peak_hbm_gbs"] = pk["hbm_gbs"]
        line["decode_batched"] = decode_batched(torch, api, (8, 16), LAYERS, pk["hbm_gbs"])
        line["front_end"] = front_end_bench(torch, api, pk["hbm_gbs"])
    if not args.no_decode:
        # The 100,000-token prefill in 2048-token chunks, one layer timed, same partition
        pf = None
        torch.cuda.empty_cache()
        part = None
        if q_shards > 1:
            n_long = (100000 + CHUNK - 1) // CHUNK
            part = lambda ci, n: q_part(ci, n, n_long)  # noqa: E731
        long_tokens = 100000
        long_splits = [slices_at(p0) for p0 in range(0, long_tokens, CHUNK)]
        ms_layer, long_parity = prefill_long(torch, api, long_tokens, heads_local, n_kv_local, part,
                                             key_splits=max(long_splits), kv_seed=4 + 1000 * kv_index,
                                             slices_at=slices_at)
        ms_layer = rank_max(ms_layer)
        long_parity["max_abs"] = rank_max(long_parity["max_abs"])
        long_parity["rel_l2"] = rank_max(long_parity["rel_l2"])
        long_parity["ranks_checked"] = world
        flop_layer = attn_flops(chunk_pairs(0, long_tokens))
        line["long_context_prefill"] = {
            "tokens": long_tokens, "chunk": CHUNK, "layers_timed": 1, "ms_per_layer": ms_layer,
            "key_slices_by_chunk": "".join(str(x) for x in long_splits),
            "tok_s_16_layers": long_tokens / (LAYERS * ms_layer * 1e-3),
            "algorithmic_tflops_all_gpus": flop_layer / (ms_layer * 1e-3) / 1e12,
            "frac_of_peak_all_gpus": flop_layer / (ms_layer * 1e-3) / 1e12 / (pk["tflops"] * world),
            "parity": long_parity}
    if world > 1 and not args.no_decode:
        torch.cuda.empty_cache()
        line["decode"] = [decode_sharded(torch, dist, api, 100000, DECODE_STEPS, LAYERS, world, rank,
                                         pk["hbm_gbs"])]
        line["decode_peak_hbm_gbs"] = pk["hbm_gbs"]
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------------- reference arm

def reference_main(args):
    """The reference's CPU attention (oracle port; the Rust original cannot be built here)
    on all host cores: each step is a bounded sample of the same prefill workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np

    import oracle as O
    cores = os.cpu_count() or 1
    rng = np.random.default_rng(1)
    tokens = T_PREFILL
    q = rng.standard_normal((tokens, QW), dtype=np.float32)
    kf = rng.standard_normal((KV, tokens, D), dtype=np.float32)
    vf = rng.standard_normal((KV, tokens, D), dtype=np.float32)
    # q8_0 cache as the engine holds it; the oracle attends over the dequantised values
    kq = O.dequantize_q8(O.quantize_q8(kf)).reshape(KV, tokens, D).transpose(1, 0, 2).reshape(tokens, W)
    vq = O.dequantize_q8(O.quantize_q8(vf)).reshape(KV, tokens, D).transpose(1, 0, 2).reshape(tokens, W)
    # 1024 rows per step (a few seconds on all threads), a whole number of rounds of the threads
    n_rows = cores * ((1024 + cores - 1) // cores)
    step = max(tokens // n_rows, 1)
    row0 = step // 2
    rows = np.arange(row0, tokens, step)
    pairs_sample = int(sum(r + 1 for r in rows))
    pairs_full = chunk_pairs(0, tokens)

    def one():
        t0 = time.perf_counter()
        O.attn_chunk_f32(q, kq, vq, H, KV, D, 0, tokens, SCALE, row0=row0, row_step=step,
                         threads=cores)
        return time.perf_counter() - t0

    for _ in range(args.warmup):
        one()
    dts = [one() for _ in range(args.steps)]
    dt = sum(dts) / len(dts)
    t_layer = dt * pairs_full / pairs_sample
    tok_s = tokens / (LAYERS * t_layer)
    sample = (f"{len(rows)} evenly spaced query rows x 24 heads of one layer per step on {cores} "
              f"threads ({dt:.2f} s per step measured), scaled by causal pair count to 16 layers")
    print(json.dumps({
        "impl": "reference", "metric": "attn prefill tok/s", "value": tok_s, "unit": "tok/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": LAYERS * t_layer * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic N(0,1), seeded",
        "config": {"workload": WORKLOAD, "l2": L2_NOTE},
        "sampled_rows_per_step": int(len(rows)), "sampled_seconds_per_step": dt,
        "sampled_seconds_total": float(sum(dts)),
        "ms_per_step_is": "extrapolated from the sampled rows by causal pair count",
        "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def profile_case(args):
    """Small single-kernel cases for `ncu` captures (a few launches, a few hundred MB held):
    chunk  -- one 2048-token chunk at position 6144 of one layer (the largest chunk of the
              headline workload): kv_encode_bulk, stage, attn_chunk_tc, `--reps` times;
    decode -- one layer's decode at depth 100000 (217.6 MB of q8 K/V, larger than L2):
              kv_encode_q8, attn_decode_kv_tc, attn_decode_kv_reduce, `--reps` times
              (`--selector 1`: the same over a q4_0 cache, 115.2 MB);
    batched -- one layer of the 16-slot batched decode step (mixed depths 615..7824).
    Prints the CUDA-event time per repetition so the capture has an un-profiled number."""
    import torch

    import __graft_entry__ as entry
    entry.build()
    from hipml_b200 import api
    torch.cuda.set_device(0)
    api.set_decode_fold_mode(args.fold_mode)
    if args.body:
        api.set_decode_body(args.body)
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(7)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * args.reps)]
    if args.case == "decode_steps":
        # the decode section of the benchmark alone: 128 graph-captured steps x 16 layers per depth
        pk = peaks()
        depths = DECODE_DEPTHS if args.depth == 100000 and args.all_depths else (args.depth,)
        for r in decode_bench(torch, api, depths, DECODE_STEPS, LAYERS, pk["hbm_gbs"]):
            print(json.dumps(r))
        if args.all_depths:
            for r in decode_batched(torch, api, (8, 16), LAYERS, pk["hbm_gbs"]):
                print(json.dumps({k: v for k, v in r.items() if k != "depths"}))
        return
    if args.case == "front":
        r = front_end_bench(torch, api, peaks()["hbm_gbs"], reps=args.reps)
        print(json.dumps({"case": "front end of a 2048-token chunk", **r}))
        return
    if args.case == "batched":
        # one layer of the 16-slot batched decode (depths as in the benchmark, seed 3): the
        # step of hipml_attn_decode_batch_append, `--reps` times; 157 MB of live K/V rows
        import oracle as O
        slots, stride = 16, 8448
        rng = O.Rng(3)
        depths = [512 + int(rng.uniform() * 7681) for _ in range(slots)]
        slot_bytes = KV * stride * ROW
        kc = torch.zeros(slots * slot_bytes, dtype=torch.uint8, device=dev)
        vc = torch.zeros_like(kc)
        for s_, d_ in enumerate(depths):
            api.kv_encode_bulk(torch.randn(d_, W, device=dev, generator=g),
                               torch.randn(d_, W, device=dev, generator=g), kc[s_ * slot_bytes:],
                               vc[s_ * slot_bytes:], KV, D, stride, 0, 0, d_)
        splits = api.batch_splits(stride, slots)
        acc_slot, ml_slot = H * splits * D, H * splits * 2
        q = torch.randn(args.reps, slots, QW, device=dev, generator=g)
        kn = torch.randn(args.reps, slots, W, device=dev, generator=g)
        vn = torch.randn(args.reps, slots, W, device=dev, generator=g)
        out = torch.empty(args.reps, slots, QW, device=dev)
        acc = torch.empty(slots * acc_slot, device=dev)
        ml = torch.empty(slots * ml_slot, device=dev)
        pos = torch.tensor([[[d_ + r, d_ + r + 1] for d_ in depths] for r in range(args.reps)],
                           dtype=torch.int32, device=dev)
        torch.cuda.synchronize()
        for r in range(args.reps):
            ev[2 * r].record()
            api.attn_decode_batch_append(pos[r], kn[r], vn[r], q[r], kc, vc, acc, ml, out[r], H, KV, D,
                                         stride, SCALE, splits, slot_bytes, acc_slot, ml_slot, QW, slots)
            ev[2 * r + 1].record()
        torch.cuda.synchronize()
        for r in range(args.reps):
            ms = ev[2 * r].elapsed_time(ev[2 * r + 1])
            nbytes = sum(2 * KV * (d_ + r + 1) * ROW for d_ in depths)
            print(json.dumps({"case": "batched decode, 16 slots, one layer", "ms": ms,
                              "kv_gbs": nbytes / ms / 1e6}))
        return
    if args.case == "chunk":
        # --kv-heads < 4 stands for one rank's share of a KV-head-sharded job
        # --pos0 / --rows move and shorten the chunk (a rank's share of the query rows, or a
        # shallower key range, for the partition A/B of the multi-GPU notes)
        pos0, n, stride = args.pos0, args.rows, 8200
        kv, sp = args.kv_heads, args.splits
        heads, qw, w = 6 * kv, 6 * kv * D, kv * D
        q = torch.randn(n, qw, device=dev, generator=g)
        kf = torch.randn(pos0 + n, w, device=dev, generator=g)
        vf = torch.randn(pos0 + n, w, device=dev, generator=g)
        kc = torch.zeros(kv * stride * ROW, dtype=torch.uint8, device=dev)
        vc = torch.zeros_like(kc)
        out = torch.empty(n, qw, device=dev)
        cap = 8192
        ws = torch.empty(api.attn_chunk_workspace_bytes(kv, D, 0, cap), dtype=torch.uint8, device=dev)
        pa = pm = None
        if sp >= 2:
            qslots = (n + 31) // 32 * 32
            pa = torch.empty(sp * qslots * heads * D, device=dev)
            pm = torch.empty(sp * qslots * heads * 2, device=dev)
        api.kv_encode_bulk(kf, vf, kc, vc, kv, D, stride, 0, 0, pos0)
        api.attn_chunk_stage(kc, vc, kv, D, 1, stride, 0, pos0, cap, ws)
        for r in range(args.reps):
            api.kv_encode_bulk(kf[pos0:], vf[pos0:], kc, vc, kv, D, stride, pos0, 0, n)
            api.attn_chunk_stage(kc, vc, kv, D, 1, stride, pos0, pos0 + n, cap, ws)
            ev[2 * r].record()
            api.attn_chunk_staged(q, out, heads, kv, D, pos0, n, cap, ws, pa, pm, sp, mode=args.mode)
            ev[2 * r + 1].record()
        torch.cuda.synchronize()
        flops = attn_flops(chunk_pairs(pos0, n)) * kv / KV
        for r in range(args.reps):
            ms = ev[2 * r].elapsed_time(ev[2 * r + 1])
            print(json.dumps({"case": f"chunk {n}@{pos0}", "mode": args.mode, "kv_heads": kv,
                              "splits": sp, "ms": ms, "algorithmic_tflops": flops / ms / 1e9}))
    else:
        depth = args.depth
        stride = depth + 136
        # --selector 1 runs the same case over a q4_0 cache (144-byte rows)
        kvd = 1 if args.selector == 1 else 0
        row = 144 if kvd else ROW
        kc = torch.zeros(KV * stride * row, dtype=torch.uint8, device=dev)
        vc = torch.zeros_like(kc)
        for p0 in range(0, depth, 8192):
            n = min(8192, depth - p0)
            api.kv_encode_bulk(torch.randn(n, W, device=dev, generator=g),
                               torch.randn(n, W, device=dev, generator=g), kc, vc, KV, D, stride,
                               p0, 0, n, dtype=kvd)
        q = torch.randn(args.reps, QW, device=dev, generator=g)
        kn = torch.randn(args.reps, W, device=dev, generator=g)
        vn = torch.randn(args.reps, W, device=dev, generator=g)
        out = torch.empty(args.reps, QW, device=dev)
        acc = torch.empty(H * 256 * D, device=dev)
        ml = torch.empty(H * 256 * 2, device=dev)
        steps = torch.zeros(args.reps, 8, dtype=torch.int32, device=dev)
        steps[:, 0] = torch.arange(depth, depth + args.reps, dtype=torch.int32, device=dev)
        steps[:, 1] = steps[:, 0] + 1
        torch.cuda.synchronize()
        for r in range(args.reps):
            api.kv_encode(steps[r], kn[r], vn[r], kc, vc, KV, D, stride, dtype=kvd)
            ev[2 * r].record()
            api.attn_decode_kv(steps[r], q[r], kc, vc, acc, ml, out[r], H, KV, D, stride, SCALE,
                               api.decode_splits(depth + r + 1), selector=args.selector)
            ev[2 * r + 1].record()
        torch.cuda.synchronize()
        for r in range(args.reps):
            ms = ev[2 * r].elapsed_time(ev[2 * r + 1])
            nbytes = 2 * KV * (depth + r + 1) * row
            print(json.dumps({"case": f"decode depth {depth}", "selector": args.selector, "ms": ms,
                              "kv_gbs": nbytes / ms / 1e6}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", choices=["chunk", "decode", "front", "batched", "decode_steps"], default=None,
                    help="run one small profiling case instead of the benchmark")
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--mode", type=int, default=0)
    ap.add_argument("--splits", type=int, default=1)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--pos0", type=int, default=6144, help="chunk case: position of the chunk's first row")
    ap.add_argument("--rows", type=int, default=2048, help="chunk case: query rows of the chunk")
    ap.add_argument("--selector", type=int, default=0)
    ap.add_argument("--depth", type=int, default=100000)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="hipml_b200")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--query-partition", choices=["chunks", "rows"], default="chunks",
                    help="N = 8: the ranks that share a KV head split the prefill by chunk pairs "
                         "(i, n-1-i) or by rotating halves of every chunk's rows")
    ap.add_argument("--decode-only", action="store_true", help="N > 1: only the sequence-split decode leg")
    ap.add_argument("--all-depths", action="store_true", help="decode_steps: every depth and the batched cases")
    ap.add_argument("--body", type=int, default=0, help="decode cases: 1 values on mma.sync, 2 on tcgen05")
    ap.add_argument("--fold-mode", type=int, default=0, help="decode cases: 1 = the fold as its own launch")
    args = ap.parse_args()
    if args.case:
        profile_case(args)
    elif args.impl == "reference":
        reference_main(args)
    else:
        gpu_main(args)


if __name__ == "__main__":
    main()
