"""The reference's kernels, recompiled for sm_100a, timed beside this library's on the same operands.

wiketool/ToyInfer's program cannot be built here (its third_party sources are absent), but its
kernels can: ``ref_kernels_shim.cu`` includes the reference's ``src/kernel.cu`` unchanged and
exports its own wrappers (include/kernel_warpper.h).  The reference's ``src/`` and ``include/``
are expected under ``baseline/_ref/`` (copied there by hand; the folder is not part of the
repository); without them every case reports ``unavailable``.

    python bench.py --kernel ref:all            (or ref:gemv_qkv, ref:flash_attention_256, ...)

Each case runs both kernels back to back from CUDA graphs over operand sets that together
exceed the L2, times them with CUDA events, and also reports the largest difference between the
two results (they compute the same thing from the same bfloat16 operands).
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
H, I, V = 2560, 9728, 151936            # Qwen3-4B layer sizes
NH, NKV, HD = 32, 8, 128

GEMV = {"gemv_qkv": (6144, H), "gemv_o": (H, 4096), "gemv_gate_up": (2 * I, H), "gemv_down": (H, I), "gemv_head": (V, H)}
BATCH = {"batch_gemv_qkv_256": (256, 6144, H), "batch_gemv_gate_up_256": (256, 2 * I, H), "batch_gemv_down_256": (256, H, I)}
FLASH = {"flash_attention_256": 256, "flash_attention_2048": 2048}
DECODE = {"attention_decode_2048": 2048, "attention_decode_8192": 8192}
CASES = list(GEMV) + list(BATCH) + list(FLASH) + list(DECODE)


def available() -> str:
    """Empty when the reference's sources are in place, else the reason."""
    if not os.path.isfile(os.path.join(REF, "src", "kernel.cu")):
        return "the reference's src/ and include/ are not under baseline/_ref/"
    return ""


def build() -> ctypes.CDLL:
    out_dir = os.path.join(HERE, "_build")
    os.makedirs(out_dir, exist_ok=True)
    lib = os.path.join(out_dir, "libref_kernels.so")
    src = os.path.join(HERE, "ref_kernels_shim.cu")
    if not os.path.isfile(lib) or os.path.getmtime(lib) < os.path.getmtime(src):
        print("[ref_kernels] compiling the reference's kernels for sm_100a", file=sys.stderr, flush=True)
        cmd = ["nvcc", "-shared", "-o", lib, src, "-I", os.path.join(REF, "src"), "-I", os.path.join(REF, "include"),
               "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-w"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"the reference's kernels did not compile:\n{r.stderr}")
    dll = ctypes.CDLL(lib)
    P, U = ctypes.c_void_p, ctypes.c_uint
    dll.ref_gemv.argtypes = [P, P, P, U, U, P]
    dll.ref_gemv_f32.argtypes = [P, P, P, U, U, P]
    dll.ref_batch_gemv.argtypes = [P, P, P, U, U, U, P]
    dll.ref_flash_attention.argtypes = [P, P, P, P, U, U, U, U, P]
    dll.ref_attention_decode.argtypes = [P, P, P, P, P, P, U, U, U, U, U, P]
    for f in (dll.ref_gemv, dll.ref_gemv_f32, dll.ref_batch_gemv, dll.ref_flash_attention, dll.ref_attention_decode):
        f.restype = None
    return dll


def _time(calls, reps):
    """ms per call of the given closures, replayed from one CUDA graph."""
    import torch
    for f in calls:
        f()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for f in calls:
            f()
    graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / (reps * len(calls))


def run(case: str, reps: int = 10) -> dict:
    import torch
    import toyinfer_b200.kernels as K
    from toyinfer_b200.cache.manager import KVView
    from toyinfer_b200.engine.batch import BatchBuffers, fill_batch

    why = available()
    if why:
        return {"kernel": "ref:" + case, "unavailable": why}
    dll = build()
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, generator=g, device=dev) * scale).to(torch.bfloat16)

    def n_sets(nbytes):
        return max(1, min(16, math.ceil(400e6 / nbytes)))

    ours, theirs, pairs, note, nbytes, flops = [], [], [], "", 0, 0.0
    if case in GEMV:
        N, Kd = GEMV[case]
        nbytes, flops = N * Kd * 2, 2.0 * N * Kd
        f32 = case == "gemv_head"
        for _ in range(n_sets(nbytes)):
            w, x = rnd(N, Kd, scale=0.02), rnd(1, Kd)
            y = torch.empty(N, dtype=torch.float32 if f32 else torch.bfloat16, device=dev)
            fn = dll.ref_gemv_f32 if f32 else dll.ref_gemv
            theirs.append(lambda w=w, x=x, y=y, fn=fn: fn(ptr(w), ptr(x), ptr(y), N, Kd, stream()))
            o = [None]
            ours.append(lambda w=w, x=x, o=o: o.__setitem__(0, K.linear(x, w, out_dtype=torch.float32 if f32 else None)))
            pairs.append((o, y))
        note = "one token; the reference runs q, k, v (and gate, up) as separate products, here its kernel gets them as one matrix"
    elif case in BATCH:
        T, N, Kd = BATCH[case]
        nbytes, flops = (N * Kd + T * Kd + T * N) * 2, 2.0 * T * N * Kd
        for _ in range(n_sets(nbytes)):
            w, x = rnd(N, Kd, scale=0.02), rnd(T, Kd)
            y = torch.empty(T, N, dtype=torch.bfloat16, device=dev)
            theirs.append(lambda w=w, x=x, y=y: dll.ref_batch_gemv(ptr(w), ptr(x), ptr(y), T, N, Kd, stream()))
            o = [None]
            ours.append(lambda w=w, x=x, o=o: o.__setitem__(0, K.linear(x, w)))
            pairs.append((o, y))
        note = f"{T} tokens: the reference's grid is (rows, tokens), one block per output element"
    elif case in FLASH:
        T = FLASH[case]
        nbytes, flops = T * (NH + 2 * NKV) * HD * 2 + T * NH * HD * 2, 4.0 * NH * HD * T * (T + 1) / 2
        batch = fill_batch(BatchBuffers(1, T, dev), "start", [0], [0], [[0] * T], 1, T)
        for _ in range(n_sets(nbytes)):
            q, k, v = rnd(T, NH, HD), rnd(T, NKV, HD), rnd(T, NKV, HD)
            y = torch.empty(T, NH, HD, dtype=torch.bfloat16, device=dev)
            theirs.append(lambda q=q, k=k, v=v, y=y: dll.ref_flash_attention(ptr(q), ptr(k), ptr(v), ptr(y), NH, NKV, HD, T, stream()))
            o = [None]
            ours.append(lambda q=q, k=k, v=v, o=o: o.__setitem__(0, K.attention_prefill(q, k, v, 1 / math.sqrt(HD), 0, batch)))
            pairs.append((o, y))
        note = f"one prompt of {T} tokens, 32 heads over 8 kv heads of 128; flops count the causal half"
    elif case in DECODE:
        L = DECODE[case]
        nbytes, flops = 2 * L * NKV * HD * 2, 4.0 * L * NH * HD
        pages = L // 64
        batch = fill_batch(BatchBuffers(1, 1, dev), "extend", [0], [L - 1], [[0]], 1, L)
        for _ in range(n_sets(nbytes)):
            ks, vs, q = rnd(L, NKV, HD), rnd(L, NKV, HD), rnd(1, NH, HD)
            score = torch.empty(NH * L, dtype=torch.float32, device=dev)
            obuf = torch.empty(NH * HD, dtype=torch.float32, device=dev)
            y = torch.empty(1, NH, HD, dtype=torch.bfloat16, device=dev)
            theirs.append(lambda q=q, ks=ks, vs=vs, score=score, obuf=obuf, y=y: dll.ref_attention_decode(
                ptr(q), ptr(ks), ptr(vs), ptr(score), ptr(obuf), ptr(y), NH, NKV, HD, L - 1, L, stream()))
            # the same keys and values in this library's layout: pages of 64 positions per kv head
            kp = torch.zeros(pages + 1, NKV, 64, HD, dtype=torch.bfloat16, device=dev)
            vp = torch.zeros_like(kp)
            kp[1:] = ks.view(pages, 64, NKV, HD).transpose(1, 2)
            vp[1:] = vs.view(pages, 64, NKV, HD).transpose(1, 2)
            table = torch.zeros(2, pages, dtype=torch.int32, device=dev)
            table[0] = torch.arange(1, pages + 1, dtype=torch.int32, device=dev)
            mem = KVView(kp, vp, table, NKV, HD, 0, 0)
            o = [None]
            ours.append(lambda q=q, mem=mem, o=o: o.__setitem__(0, K.attention_decode(q, mem, 1 / math.sqrt(HD), 0, batch)))
            pairs.append((o, y))
        note = f"one sequence of {L} positions; the reference's chain is two memsets and four kernels, this library's two kernels"
    else:
        raise SystemExit(f"unknown reference case {case!r}; cases: {', '.join(CASES)}")

    ms_ref = _time(theirs, reps)
    ms_ours = _time(ours, reps)
    K.check_status()
    diff = max(float((o[0].float().reshape(-1) - y.float().reshape(-1)).abs().max()) for o, y in pairs)
    scale = max(float(y.float().abs().max()) for _, y in pairs)
    return {"kernel": "ref:" + case, "ref_ms": round(ms_ref, 4), "ours_ms": round(ms_ours, 4),
            "speedup": round(ms_ref / ms_ours, 2), "ref_gbs": round(nbytes / ms_ref / 1e6, 1),
            "ours_gbs": round(nbytes / ms_ours / 1e6, 1), "ref_tflops": round(flops / ms_ref / 1e9, 2),
            "ours_tflops": round(flops / ms_ours / 1e9, 2), "max_abs_diff": round(diff, 5), "max_abs_value": round(scale, 3),
            "operand_sets": len(ours), "note": note}
