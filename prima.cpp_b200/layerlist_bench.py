"""Throughput of the layer-list family at sizes that resemble a real model's layers, random weights, beside the closest existing model at
equal width / feed-forward / head sizes / number of layer runs: Vamidra beside the Llama graph over Q4_K weights (``bench.py --arch
vamidra``), Mumizen beside Vamidra (``bench.py --arch mumizen``, :func:`run_mumizen`), Sapudra beside Vamidra and, for its experts, Mumizen
(``bench.py --arch sapudra``, :func:`run_sapudra`), Zevedra beside Vamidra (attention, convolution, plain products) and Mumizen (recurrence,
experts) (``bench.py --arch zevedra``, :func:`run_zevedra`).  Prints one JSON line.

Per size: prompt tokens/s (one sequence of 512 and 2048 tokens) and decode tokens/s (batch 1 and 8 at a 1024-token context) of both
models through their public entry points (host token ids in, host logits / greedy tokens out), the device time of a prompt and of a
decode step by kernel category, the like-for-like single-op probes (prompt product: tcgen05 bf16 dense vs tcgen05 k-quant; decode
product: bf16 weight streaming vs k-quant GEMV) and every kernel's distance from its roofline (measured peaks of MEASURED_PEAKS.json).
"""
from __future__ import annotations

import ctypes as C
import json
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

SIZES = {
    "w2048": dict(width=2048, ff=8192, heads=16, kv_heads=4, dim=128, window=1024, keep_first=64, ssm_heads=32, vdim=128, state=128, groups=4,
                  conv=4, norm_groups=4, vocab=32000),
    "w4096": dict(width=4096, ff=14336, heads=32, kv_heads=8, dim=128, window=1024, keep_first=64, ssm_heads=64, vdim=128, state=128, groups=8,
                  conv=4, norm_groups=8, vocab=32000),
}


def vamidra_config(s):
    att = {"type": "attention", "mixer": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5,
                                           "softcap": 50.0, "mask": {"size": s["window"], "keep_first": s["keep_first"]}},
           "mlp": {"kind": "dense", "ff": s["ff"]}}
    ssm = {"type": "mamba2", "mixer": {"heads": s["ssm_heads"], "vdim": s["vdim"], "state": s["state"], "groups": s["groups"], "conv": s["conv"],
                                        "norm_groups": s["norm_groups"]}, "mlp": {"kind": "dense", "ff": s["ff"]}}
    # attention, mamba2 repeated twice with shared weights, then one more pair: 6 layer runs
    return {"architecture": "Vamidra", "width": s["width"], "vocab": s["vocab"], "logit_scale": 1.0, "norm": {"eps": 1e-6},
            "layers": [att, ssm, dict(att), dict(ssm)], "loop": {"start": 0, "stop": 2, "times": 2}}


def dense_shapes(s, cfg):
    """(N, K) of every dense product of one token through all layer runs (the head not included)."""
    W, out = s["width"], []
    order = [0, 1, 0, 1, 2, 3]
    for t, li in enumerate(order):
        if li == 0:
            out += [(W, W), (W, W)]                                        # input mix of a pass: two halves
        m = cfg["layers"][li]["mixer"]
        if cfg["layers"][li]["type"] == "attention":
            out += [(m["heads"] * m["dim"] + 2 * m["kv_heads"] * m["dim"] + m["heads"], W), (W, m["heads"] * m["vdim"])]
        else:
            inner = m["heads"] * m["vdim"]
            out += [(2 * inner + 2 * m["groups"] * m["state"] + m["heads"], W), (W, inner)]
        out += [(2 * s["ff"], W), (W, s["ff"])]
    return out


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


def run(args, pkg, lib):
    if args.arch == "mumizen":
        return run_mumizen(args, pkg, lib)
    if args.arch == "sapudra":
        return run_sapudra(args, pkg, lib)
    if args.arch == "zevedra":
        return run_zevedra(args, pkg, lib)
    import numpy as np
    import torch
    hbm, tflops, src = peaks()
    ptr = lambda t: C.c_void_p(t.data_ptr())   # noqa: E731
    sync = torch.cuda.synchronize
    res = {"metric": "Vamidra prompt / decode throughput beside the Llama graph at equal size", "impl": "b200", "arch": "Vamidra", "n_gpus": 1,
           "dtype": "bf16", "data": "synthetic random weights", "peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": src}, "sizes": {}}
    rng = np.random.default_rng(0)

    def timed(fn, reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        sync()
        return e0.elapsed_time(e1) / reps

    for key in ([args.arch_size] if args.arch_size != "all" else list(SIZES)):
        s = SIZES[key]
        cfg = vamidra_config(s)
        out = {"config": {k: s[k] for k in ("width", "ff", "heads", "kv_heads", "window", "keep_first", "ssm_heads", "state")}, "layer_runs": 6}
        # ---------------- the new design ----------------
        m = pkg.Model.from_config(cfg, dtype="bfloat16", n_ctx=4096, n_seq=16)
        m.synth(0, 7)
        m.finalize()
        shapes = dense_shapes(s, cfg)
        flops_tok = 2.0 * sum(n * k for n, k in shapes)
        wbytes = 2.0 * sum(n * k for n, k in shapes) + 2.0 * s["vocab"] * s["width"]
        v = {}
        for T in (512, 2048):
            toks = rng.integers(0, s["vocab"], T).tolist()

            def prompt():
                sl = m.seq_alloc()
                m.batch_step([(sl, toks, [T - 1])])
                m.seq_free(sl)
            for _ in range(3):
                prompt()
            t0 = time.perf_counter()
            reps = max(3, args.steps // 16)
            for _ in range(reps):
                prompt()
            dt = (time.perf_counter() - t0) / reps
            v[f"prompt{T}_tok_s"] = T / dt
            m.profile(True)
            prompt()
            pm = m.profile_ms()
            m.profile(False)
            v[f"prompt{T}_device_ms"] = pm
            v[f"prompt{T}_dense_tflops"] = flops_tok * T / pm["dense"] / 1e9
            v[f"prompt{T}_dense_frac_of_tensor_peak"] = v[f"prompt{T}_dense_tflops"] / tflops
            # attention: 4 * dim * visible keys per query and head; 3 attention runs
            vis = sum(min(i + 1, s["window"]) + max(0, min(s["keep_first"], i + 1 - s["window"])) for i in range(T))
            v[f"prompt{T}_attention_tflops"] = 3 * 4.0 * s["dim"] * s["heads"] * vis / pm["attention"] / 1e9
            # scan: bytes that must move (conv outputs read, y written, step sizes), 3 mamba runs
            inner, ch = s["ssm_heads"] * s["vdim"], s["ssm_heads"] * s["vdim"] + 2 * s["groups"] * s["state"]
            v[f"prompt{T}_scan_gbs"] = 3 * T * 4.0 * (ch + inner + s["ssm_heads"]) / pm["scan"] / 1e6
            v[f"prompt{T}_scan_gflops"] = 3 * T * 6.0 * s["ssm_heads"] * s["state"] * s["vdim"] / pm["scan"] / 1e6
        for B in (1, 8):
            slots = [m.seq_alloc() for _ in range(B)]
            ctx = rng.integers(0, s["vocab"], 1024).tolist()
            m.batch_step([(sl, ctx, []) for sl in slots])
            step = lambda: m.batch_step([(sl, [5], []) for sl in slots], greedy=True)   # noqa: E731
            for _ in range(max(3, args.warmup)):
                step()
            t0 = time.perf_counter()
            for _ in range(args.steps):
                step()
            dt = (time.perf_counter() - t0) / args.steps
            v[f"decode_b{B}_tok_s"] = B / dt
            v[f"decode_b{B}_ms_per_step"] = dt * 1e3
            v[f"decode_b{B}_whole_step_frac_of_hbm_peak"] = wbytes / dt / 1e9 / hbm
            m.profile(True)
            step()
            pm = m.profile_ms()
            m.profile(False)
            v[f"decode_b{B}_device_ms"] = pm
            v[f"decode_b{B}_dense_gbs"] = (wbytes - 2.0 * s["vocab"] * s["width"]) / pm["dense"] / 1e6
            v[f"decode_b{B}_dense_frac_of_hbm_peak"] = v[f"decode_b{B}_dense_gbs"] / hbm
            for sl in slots:
                m.seq_free(sl)
        v["weight_bytes_per_token"] = wbytes
        m.close()
        out["vamidra"] = v
        # ---------------- the closest existing model: the Llama graph, Q4_K, equal sizes, 6 layers ----------------
        hp = pkg.HParams(n_layer=6, n_embd=s["width"], n_head=s["heads"], n_head_kv=s["kv_heads"], head_dim=128, n_ff=s["ff"], n_vocab=s["vocab"],
                         n_ctx=4096, rope_mode=0, n_ctx_orig=8192, rope_freq_base=500000.0, rope_freq_scale=1.0, rms_eps=1e-5)
        eng = pkg.Model(hp)
        eng.synth(0, 11)
        eng.finalize()
        w = {}
        logits = np.empty(s["vocab"], dtype=np.float32)
        for T in (512, 2048):
            toks = rng.integers(0, s["vocab"], T).astype(np.int32)
            for _ in range(3):
                eng.prefill(toks, 0, logits)
            t0 = time.perf_counter()
            reps = max(3, args.steps // 16)
            for _ in range(reps):
                eng.prefill(toks, 0, logits)
            w[f"prompt{T}_tok_s"] = T / ((time.perf_counter() - t0) / reps)
        eng.prefill(rng.integers(0, s["vocab"], 1024).astype(np.int32), 0, logits)
        for i in range(max(3, args.warmup)):
            eng.decode(5, 1024 + i, logits)
        t0 = time.perf_counter()
        for i in range(args.steps):
            eng.decode(5, 1100 + i, logits)
        dt = (time.perf_counter() - t0) / args.steps
        w["decode_b1_tok_s"] = 1.0 / dt
        w["decode_b1_whole_step_frac_of_hbm_peak"] = eng.weight_bytes / dt / 1e9 / hbm
        pr = eng.profile_step(5, 1300)
        w["decode_b1_gemv_gbs"] = pr["gemv_bytes"] / pr["gemv_ms"] / 1e6
        w["decode_b1_gemv_frac_of_hbm_peak"] = w["decode_b1_gemv_gbs"] / hbm
        w["weight_bytes_per_token"] = eng.weight_bytes
        eng.close()
        out["llama_q4_k"] = w
        # ---------------- like-for-like single-op probes at the feed-forward shapes ----------------
        probes = {}
        for name, (N, K) in (("gate_up", (2 * s["ff"], s["width"])), ("down", (s["width"], s["ff"]))):
            for T in (512, 2048):
                A = torch.randn((T, K), device="cuda").to(torch.bfloat16)
                Wd = (torch.randn((N, K), device="cuda") / K ** 0.5).to(torch.bfloat16)
                Cd = torch.empty((T, N), device="cuda")
                f = lambda: lib.c.pb200_dense(30, ptr(A), K, ptr(Wd), K, ptr(Cd), N, T, N, K, None, None, 0, 1.0, None)   # noqa: E731
                for _ in range(3):
                    f()
                ms = timed(f, 10)
                rb = lib.c.pb200_row_bytes(12, K)
                Wq = torch.randint(0, 255, (N * rb + 64,), dtype=torch.uint8, device="cuda")
                xd = torch.randn((T, K), device="cuda")
                ws = torch.zeros(lib.c.pb200_mul_mat_q_workspace_bytes(K, T) + 64, dtype=torch.uint8, device="cuda")
                g = lambda: lib.c.pb200_mul_mat_q(12, ptr(Wq), N, K, ptr(xd), K, T, ptr(Cd), None, None, ptr(ws), None)   # noqa: E731
                for _ in range(3):
                    g()
                ms_q = timed(g, 10)
                fl = 2.0 * N * K * T
                probes[f"prompt_product_{name}_T{T}"] = {"dense_bf16_tflops": fl / ms / 1e9, "dense_bf16_frac_of_tensor_peak": fl / ms / 1e9 / tflops,
                                                         "kquant_q4_K_tflops": fl / ms_q / 1e9, "kquant_q4_K_frac_of_tensor_peak": fl / ms_q / 1e9 / tflops}
                del A, Wd, Cd, Wq, xd, ws
            # decode product: weights larger than L2 are streamed once per call
            for T in (1, 8):
                A = torch.randn((T, K), device="cuda").to(torch.bfloat16)
                Wd = (torch.randn((N, K), device="cuda") / K ** 0.5).to(torch.bfloat16)
                Cd = torch.empty((T, N), device="cuda")
                f = lambda: lib.c.pb200_dense(30, ptr(A), K, ptr(Wd), K, ptr(Cd), N, T, N, K, None, None, 0, 1.0, None)   # noqa: E731
                for _ in range(3):
                    f()
                ms = timed(f, 20)
                probes[f"decode_product_{name}_b{T}"] = {"dense_bf16_gbs": 2.0 * N * K / ms / 1e6, "dense_bf16_frac_of_hbm_peak": 2.0 * N * K / ms / 1e6 / hbm}
                if T == 1:
                    rb = lib.c.pb200_row_bytes(12, K)
                    Wq = torch.randint(0, 255, (N * rb + 64,), dtype=torch.uint8, device="cuda")
                    xd = torch.randn((K,), device="cuda")
                    yd = torch.empty((N,), device="cuda")
                    aw = torch.zeros(lib.c.pb200_act_workspace_bytes(K) + 64, dtype=torch.uint8, device="cuda")
                    g = lambda: lib.c.pb200_mul_mat_vec(12, ptr(Wq), N, K, ptr(xd), ptr(yd), ptr(aw), None)   # noqa: E731
                    for _ in range(3):
                        g()
                    ms_q = timed(g, 20)
                    probes[f"decode_product_{name}_b{T}"].update({"kquant_q4_K_gbs": N * rb / ms_q / 1e6, "kquant_q4_K_frac_of_hbm_peak": N * rb / ms_q / 1e6 / hbm})
                    del Wq, xd, yd, aw
                del A, Wd, Cd
        # prompt attention: the Llama graph's tiled kernel (every earlier position, f16 cache) against the windowed kernel's share of a prompt
        T, H, HK = 2048, s["heads"], s["kv_heads"]
        q = torch.randn((T, H * 128), device="cuda")
        kc = torch.randn((T, HK * 128), device="cuda").to(torch.float16)
        vc = torch.randn((T, HK * 128), device="cuda").to(torch.float16)
        o = torch.empty((T, H * 128), device="cuda")
        pos = torch.arange(T, dtype=torch.int32, device="cuda")
        f = lambda: lib.c.pb200_attn_prefill(ptr(q), ptr(kc), ptr(vc), ptr(o), H, HK, 128, ptr(pos), T, T, 128 ** -0.5, None)   # noqa: E731
        for _ in range(3):
            f()
        ms = timed(f, 10)
        probes["prompt_attention_T2048"] = {"llama_causal_tflops": 4.0 * 128 * H * T * (T + 1) / 2 / ms / 1e9, "llama_ms": ms,
                                            "vamidra_windowed_tflops": v["prompt2048_attention_tflops"],
                                            "vamidra_ms_per_run": v["prompt2048_device_ms"]["attention"] / 3}
        del q, kc, vc, o, pos
        out["like_kernels"] = probes
        res["sizes"][key] = out
        torch.cuda.empty_cache()
    res["gpu_launches"] = int(lib.c.pb200_kernel_launches())
    print(json.dumps(res))
    return res


# ---------------------------------------------------------------------------------------------------------------
MUMIZEN_SIZES = {
    "w2048": dict(heads=16, dim=128, vdim=128, rot_dim=64, kv_rank=512, q_rank=1024, experts=16, top=2, expert_ff=2048, shared_ff=2048, groups=4),
    "w4096": dict(heads=32, dim=128, vdim=128, rot_dim=64, kv_rank=512, q_rank=1536, experts=16, top=2, expert_ff=4096, shared_ff=4096, groups=8),
}


def mumizen_config(s, z):
    """Six layers at the width / feed-forward of SIZES: decay attention of both kinds and latent attention (one layer reads another's
    latent cache), four dense feed-forwards and two mixtures of experts with a shared expert."""
    H = z["heads"]
    decay = [1.0 - 2.0 ** (-5 - 7 * h / max(H - 1, 1)) for h in range(H)]
    lin = {"heads": H, "dim": z["dim"], "vdim": z["vdim"], "decay": decay}
    lat = {"heads": H, "dim": z["dim"], "rot_dim": z["rot_dim"], "vdim": z["vdim"], "kv_rank": z["kv_rank"], "q_rank": z["q_rank"],
           "scale": (z["dim"] + z["rot_dim"]) ** -0.5,
           "rot": {"base": 10000.0, "dims": z["rot_dim"], "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    dense = {"kind": "dense", "ff": s["ff"], "limit": 7.0}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"], "limit": 7.0}, "router": {"experts": z["experts"], "top": z["top"]},
           "shared": {"ff": z["shared_ff"], "limit": 7.0}}
    layers = [{"type": "retention", "mixer": lin, "mlp": dense}, {"type": "lightning", "mixer": lin, "mlp": moe},
              {"type": "latent_attention", "mixer": lat, "mlp": dense}, {"type": "latent_attention", "mixer": dict(lat, kv_from=2), "mlp": moe},
              {"type": "lightning", "mixer": lin, "mlp": dense}, {"type": "latent_attention", "mixer": lat, "mlp": dense}]
    return {"architecture": "Mumizen", "width": s["width"], "vocab": s["vocab"], "norm": {"eps": 1e-6, "groups": z["groups"]}, "layers": layers}


def mumizen_products(cfg, prompt):
    """((N, K) of the plain dense products, expert weight elements touched) of one token through all layers, the head not included."""
    W, out, expert = cfg["width"], [], 0
    for l in cfg["layers"]:
        m = l["mixer"]
        if l["type"] in ("lightning", "retention"):
            out += [(2 * m["heads"] * m["dim"] + 2 * m["heads"] * m["vdim"], W), (W, m["heads"] * m["vdim"])]
        else:
            H = m["heads"]
            out += [(m["q_rank"] + H * m["vdim"] + (0 if "kv_from" in m else m["kv_rank"] + m["rot_dim"]), W), (H * (m["dim"] + m["rot_dim"]), m["q_rank"]),
                    (W, H * m["vdim"])]
            if prompt:
                out += [(H * m["dim"], m["kv_rank"]), (H * m["vdim"], m["kv_rank"])]
        f = l["mlp"]
        if f["kind"] == "dense":
            out += [(2 * f["ff"], W), (W, f["ff"])]
        else:
            out += [(2 * f["shared"]["ff"], W), (W, f["shared"]["ff"])]
            expert += f["router"]["top"] * 3 * f["expert"]["ff"] * W
    return out, expert


def measure(m, vocab, args, rng, CTX=1024):
    """Whole-model prompt (512 / 2048 tokens) and decode (batch 1 / 8 at a CTX-token context) throughput through the public entry points, with the
    device time of one prompt and one step by kernel category."""
    v = {}
    for T in (512, 2048):
        toks = rng.integers(0, vocab, T).tolist()

        def prompt():
            sl = m.seq_alloc()
            m.batch_step([(sl, toks, [T - 1])])
            m.seq_free(sl)
        for _ in range(3):
            prompt()
        reps = max(3, args.steps // 16)
        t0 = time.perf_counter()
        for _ in range(reps):
            prompt()
        v[f"prompt{T}_tok_s"] = T / ((time.perf_counter() - t0) / reps)
        m.profile(True)
        prompt()
        v[f"prompt{T}_device_ms"] = m.profile_ms()
        m.profile(False)
    for B in (1, 8):
        slots = [m.seq_alloc() for _ in range(B)]
        ctx = rng.integers(0, vocab, CTX).tolist()
        m.batch_step([(sl, ctx, []) for sl in slots])
        step = lambda: m.batch_step([(sl, [5], []) for sl in slots], greedy=True)   # noqa: E731
        for _ in range(max(3, args.warmup)):
            step()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step()
        dt = (time.perf_counter() - t0) / args.steps
        v[f"decode_b{B}_tok_s"] = B / dt
        v[f"decode_b{B}_ms_per_step"] = dt * 1e3
        m.profile(True)
        step()
        v[f"decode_b{B}_device_ms"] = m.profile_ms()
        m.profile(False)
        for sl in slots:
            m.seq_free(sl)
    return v


def run_mumizen(args, pkg, lib):
    """Mumizen beside Vamidra at equal width / feed-forward / head size and six layer runs each: whole-model prompt and decode throughput
    through the public entry points, device time per kernel category, and for every pair of like kernels the distance from its roofline."""
    import numpy as np
    import torch
    hbm, tflops, src = peaks()
    res = {"metric": "Mumizen prompt / decode throughput beside Vamidra at equal size", "impl": "b200", "arch": "Mumizen", "n_gpus": 1, "dtype": "bf16",
           "data": "synthetic random weights", "peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": src}, "sizes": {}}
    rng = np.random.default_rng(0)
    CTX = 1024

    for key in ([args.arch_size] if args.arch_size != "all" else list(SIZES)):
        s, z = SIZES[key], MUMIZEN_SIZES[key]
        W, V = s["width"], s["vocab"]
        out = {"config": dict(z, width=W, ff=s["ff"], vocab=V), "layers": 6}
        # ---------------- the new design ----------------
        cfg = mumizen_config(s, z)
        m = pkg.Model.from_config(cfg, dtype="bfloat16", n_ctx=4096, n_seq=16)
        m.synth(0, 7)
        m.finalize()
        a = measure(m, V, args, rng, CTX)
        m.close()
        H, D, Dv, Dr, R = z["heads"], z["dim"], z["vdim"], z["rot_dim"], z["kv_rank"]
        n_lin = sum(l["type"] != "latent_attention" for l in cfg["layers"])
        n_lat = 6 - n_lin
        n_norm = 6 + 6 + sum(1 for l in cfg["layers"])      # norm1 (+ shift) and norm2 per layer; the depth average rides in `elementwise`
        for T in (512, 2048):
            pm = a[f"prompt{T}_device_ms"]
            prods, expert = mumizen_products(cfg, True)
            fl = 2.0 * sum(n * k for n, k in prods) * T
            a[f"prompt{T}_dense_frac_of_tensor_peak"] = fl / pm["dense"] / 1e9 / tflops
            a[f"prompt{T}_experts_frac_of_tensor_peak"] = 2.0 * expert * T / pm["experts"] / 1e9 / tflops
            a[f"prompt{T}_attention_tflops"] = n_lat * 2.0 * (D + Dr + Dv) * H * T * (T + 1) / 2 / pm["attention"] / 1e9
            a[f"prompt{T}_scan_state_updates_per_ns"] = n_lin * T * H * D * Dv / pm["scan"] / 1e6
            a[f"prompt{T}_norm_gbs"] = 12 * T * W * 6.0 / pm["norm"] / 1e6
        prods, expert = mumizen_products(cfg, False)
        wb = 2.0 * sum(n * k for n, k in prods)
        a["weight_bytes_per_token"] = wb + 2.0 * expert + 2.0 * V * W
        for B in (1, 8):
            pm = a[f"decode_b{B}_device_ms"]
            a[f"decode_b{B}_dense_frac_of_hbm_peak"] = wb / pm["dense"] / 1e6 / hbm
            a[f"decode_b{B}_experts_frac_of_hbm_peak"] = 2.0 * expert * B / pm["experts"] / 1e6 / hbm     # b = 8: the most bytes the 8 tokens can touch
            a[f"decode_b{B}_attention_gbs"] = n_lat * B * CTX * (R + Dr) * 4.0 / pm["attention"] / 1e6
            a[f"decode_b{B}_whole_step_frac_of_hbm_peak"] = a["weight_bytes_per_token"] / a[f"decode_b{B}_ms_per_step"] / 1e6 / hbm
        out["mumizen"] = a
        # ---------------- the closest existing model: Vamidra, equal sizes, 6 layer runs ----------------
        vcfg = vamidra_config(s)
        m = pkg.Model.from_config(vcfg, dtype="bfloat16", n_ctx=4096, n_seq=16)
        m.synth(0, 7)
        m.finalize()
        b = measure(m, V, args, rng, CTX)
        m.close()
        shapes = dense_shapes(s, vcfg)
        for T in (512, 2048):
            pm = b[f"prompt{T}_device_ms"]
            b[f"prompt{T}_dense_frac_of_tensor_peak"] = 2.0 * sum(n * k for n, k in shapes) * T / pm["dense"] / 1e9 / tflops
            vis = sum(min(i + 1, s["window"]) + max(0, min(s["keep_first"], i + 1 - s["window"])) for i in range(T))
            b[f"prompt{T}_attention_tflops"] = 3 * 4.0 * s["dim"] * s["heads"] * vis / pm["attention"] / 1e9
            b[f"prompt{T}_scan_state_updates_per_ns"] = 3 * T * s["ssm_heads"] * s["state"] * s["vdim"] / pm["scan"] / 1e6
            b[f"prompt{T}_norm_gbs"] = (12 * T * W * 6.0 + 3 * T * s["ssm_heads"] * s["vdim"] * 10.0) / pm["norm"] / 1e6
        wbv = 2.0 * sum(n * k for n, k in shapes)
        b["weight_bytes_per_token"] = wbv + 2.0 * V * W
        rows = min(CTX, s["window"] + s["keep_first"])
        for B in (1, 8):
            pm = b[f"decode_b{B}_device_ms"]
            b[f"decode_b{B}_dense_frac_of_hbm_peak"] = wbv / pm["dense"] / 1e6 / hbm
            b[f"decode_b{B}_attention_gbs"] = 3 * B * rows * s["kv_heads"] * 2 * s["dim"] * 4.0 / pm["attention"] / 1e6
            b[f"decode_b{B}_whole_step_frac_of_hbm_peak"] = b["weight_bytes_per_token"] / b[f"decode_b{B}_ms_per_step"] / 1e6 / hbm
        out["vamidra"] = b
        res["sizes"][key] = out
        torch.cuda.empty_cache()
    res["gpu_launches"] = int(lib.c.pb200_kernel_launches())
    print(json.dumps(res))
    return res


# ---------------------------------------------------------------------------------------------------------------
SAPUDRA_SIZES = {
    "w2048": dict(experts=16, top=2, expert_ff=2048, shared_ff=2048, count=4, keep=2),
    "w4096": dict(experts=16, top=2, expert_ff=4096, shared_ff=4096, count=4, keep=2),
}


def sapudra_config(s, z):
    """Six attention layers at the width / feed-forward / head sizes of SIZES (window as Vamidra's, no kept first tokens): four dense
    squared-ReLU feed-forwards and two mixtures of experts with a gated shared expert."""
    att = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5, "mask": {"size": s["window"]}}
    dense = {"kind": "dense", "ff": s["ff"]}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "shared": {"ff": z["shared_ff"]},
           "router": {"experts": z["experts"], "top": z["top"], "scale": 2.5, "groups": {"count": z["count"], "keep": z["keep"]}}}
    layers = [{"type": "attention", "mixer": att, "mlp": f} for f in (dense, moe, dense, moe, dense, dense)]
    return {"architecture": "Sapudra", "width": s["width"], "vocab": s["vocab"], "max_positions": 4096, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "logit_softcap": 30.0, "layers": layers}


def sapudra_products(cfg):
    """((N, K) of the plain dense products, expert weight elements touched) of one token through all layers, the head not included."""
    W, out, expert = cfg["width"], [], 0
    for l in cfg["layers"]:
        m = l["mixer"]
        out += [(m["heads"] * m["dim"] + m["kv_heads"] * (m["dim"] + m["vdim"]), W), (W, m["heads"] * m["vdim"])]
        f = l["mlp"]
        if f["kind"] == "dense":
            out += [(f["ff"], W), (W, f["ff"])]
        else:
            out += [(f["shared"]["ff"], W), (W, f["shared"]["ff"])]
            expert += f["router"]["top"] * 2 * f["expert"]["ff"] * W
    return out, expert


def run_sapudra(args, pkg, lib):
    """Sapudra beside Vamidra (attention, plain products, norms, element-wise steps: the same or like kernels) and beside Mumizen (expert
    products) at equal width / feed-forward / head size and six layer runs each: whole-model prompt and decode throughput through the
    public entry points, device time per kernel category, and for every pair of like kernels the distance from its roofline."""
    import numpy as np
    import torch
    hbm, tflops, src = peaks()
    res = {"metric": "Sapudra prompt / decode throughput beside Vamidra and Mumizen at equal size", "impl": "b200", "arch": "Sapudra", "n_gpus": 1,
           "dtype": "bf16", "data": "synthetic random weights", "peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": src}, "sizes": {}}
    rng = np.random.default_rng(0)
    CTX = 1024

    def model(cfg):
        m = pkg.Model.from_config(cfg, dtype="bfloat16", n_ctx=4096, n_seq=16)
        m.synth(0, 7)
        m.finalize()
        return m

    for key in ([args.arch_size] if args.arch_size != "all" else list(SIZES)):
        s, z = SIZES[key], SAPUDRA_SIZES[key]
        W, V, H, G, D = s["width"], s["vocab"], s["heads"], s["kv_heads"], s["dim"]
        out = {"config": dict(z, width=W, ff=s["ff"], heads=H, kv_heads=G, dim=D, window=s["window"], vocab=V), "layers": 6}
        # ---------------- the new design ----------------
        cfg = sapudra_config(s, z)
        m = model(cfg)
        a = measure(m, V, args, rng, CTX)
        m.close()
        prods, expert = sapudra_products(cfg)
        n_moe = sum(l["mlp"]["kind"] == "moe" for l in cfg["layers"])
        for T in (512, 2048):
            pm = a[f"prompt{T}_device_ms"]
            a[f"prompt{T}_dense_frac_of_tensor_peak"] = 2.0 * sum(n * k for n, k in prods) * T / pm["dense"] / 1e9 / tflops
            a[f"prompt{T}_experts_frac_of_tensor_peak"] = 2.0 * expert * T / pm["experts"] / 1e9 / tflops
            vis = sum(min(i + 1, s["window"]) for i in range(T))
            a[f"prompt{T}_attention_tflops"] = 6 * 4.0 * D * H * vis / pm["attention"] / 1e9
            # 12 post-norms: the sublayer result and x read, x and the operand written
            a[f"prompt{T}_norm_gbs"] = 12 * T * W * 14.0 / pm["norm"] / 1e6
            # squared ReLU: 4 dense + 2 shared hidden rows read (fp32) and written (bf16); embedding: table rows read, x and operand written
            elem = T * 6.0 * (4 * s["ff"] + n_moe * z["shared_ff"]) + T * W * 10.0
            a[f"prompt{T}_elementwise_gbs"] = elem / pm["elementwise"] / 1e6
        wb = 2.0 * sum(n * k for n, k in prods)
        a["weight_bytes_per_token"] = wb + 2.0 * expert + 2.0 * V * W
        rows = min(CTX, s["window"])
        for B in (1, 8):
            pm = a[f"decode_b{B}_device_ms"]
            a[f"decode_b{B}_dense_frac_of_hbm_peak"] = wb / pm["dense"] / 1e6 / hbm
            a[f"decode_b{B}_experts_frac_of_hbm_peak"] = 2.0 * expert * B / pm["experts"] / 1e6 / hbm     # b = 8: the most bytes the 8 tokens can touch
            a[f"decode_b{B}_attention_gbs"] = 6 * B * rows * G * 2 * D * 4.0 / pm["attention"] / 1e6
            a[f"decode_b{B}_whole_step_frac_of_hbm_peak"] = a["weight_bytes_per_token"] / a[f"decode_b{B}_ms_per_step"] / 1e6 / hbm
        out["sapudra"] = a
        # ---------------- the closest existing model: Vamidra, equal sizes, 6 layer runs ----------------
        vcfg = vamidra_config(s)
        m = model(vcfg)
        b = measure(m, V, args, rng, CTX)
        m.close()
        shapes = dense_shapes(s, vcfg)
        for T in (512, 2048):
            pm = b[f"prompt{T}_device_ms"]
            b[f"prompt{T}_dense_frac_of_tensor_peak"] = 2.0 * sum(n * k for n, k in shapes) * T / pm["dense"] / 1e9 / tflops
            vis = sum(min(i + 1, s["window"]) + max(0, min(s["keep_first"], i + 1 - s["window"])) for i in range(T))
            b[f"prompt{T}_attention_tflops"] = 3 * 4.0 * D * H * vis / pm["attention"] / 1e9
            b[f"prompt{T}_norm_gbs"] = (12 * T * W * 6.0 + 3 * T * s["ssm_heads"] * s["vdim"] * 10.0) / pm["norm"] / 1e6
            # tanh-GELU gating: 6 hidden rows of gate | up read (fp32), the product written (bf16); embedding; input mix casts
            b[f"prompt{T}_elementwise_gbs"] = (T * 10.0 * 6 * s["ff"] + T * W * 12.0 + 2 * 2 * T * W * 6.0) / pm["elementwise"] / 1e6
        wbv = 2.0 * sum(n * k for n, k in shapes)
        b["weight_bytes_per_token"] = wbv + 2.0 * V * W
        vrows = min(CTX, s["window"] + s["keep_first"])
        for B in (1, 8):
            pm = b[f"decode_b{B}_device_ms"]
            b[f"decode_b{B}_dense_frac_of_hbm_peak"] = wbv / pm["dense"] / 1e6 / hbm
            b[f"decode_b{B}_attention_gbs"] = 3 * B * vrows * G * 2 * D * 4.0 / pm["attention"] / 1e6
            b[f"decode_b{B}_whole_step_frac_of_hbm_peak"] = b["weight_bytes_per_token"] / b[f"decode_b{B}_ms_per_step"] / 1e6 / hbm
        out["vamidra"] = b
        # ---------------- the closest existing experts: Mumizen at equal expert sizes ----------------
        mz = dict(MUMIZEN_SIZES[key], experts=z["experts"], top=z["top"], expert_ff=z["expert_ff"], shared_ff=z["shared_ff"])
        mcfg = mumizen_config(s, mz)
        m = model(mcfg)
        c = measure(m, V, args, rng, CTX)
        m.close()
        _, mexpert = mumizen_products(mcfg, True)
        e = {}
        for T in (512, 2048):
            e[f"prompt{T}_experts_frac_of_tensor_peak"] = 2.0 * mexpert * T / c[f"prompt{T}_device_ms"]["experts"] / 1e9 / tflops
            e[f"prompt{T}_experts_ms"] = c[f"prompt{T}_device_ms"]["experts"]
        for B in (1, 8):
            e[f"decode_b{B}_experts_frac_of_hbm_peak"] = 2.0 * mexpert * B / c[f"decode_b{B}_device_ms"]["experts"] / 1e6 / hbm
            e[f"decode_b{B}_experts_ms"] = c[f"decode_b{B}_device_ms"]["experts"]
        out["mumizen_experts"] = e
        res["sizes"][key] = out
        torch.cuda.empty_cache()
    res["gpu_launches"] = int(lib.c.pb200_kernel_launches())
    print(json.dumps(res))
    return res


# ---------------------------------------------------------------------------------------------------------------
ZEVEDRA_SIZES = {
    "w2048": dict(r_heads=16, r_kv=4, r_dim=128, r_vdim=128, conv=4, experts=16, top=2, expert_ff=2048),
    "w4096": dict(r_heads=32, r_kv=8, r_dim=128, r_vdim=128, conv=4, experts=16, top=2, expert_ff=4096),
}


def zevedra_config(s, z):
    """Four layers, the first two run twice (six layer runs): sink attention beside HGRN2, then windowed attention beside the gated delta
    rule, at the width / head sizes / window of SIZES; every layer has a mixture of experts."""
    H, G, D = s["heads"], s["kv_heads"], s["dim"]
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "top": z["top"]}}
    p2 = {"type": "parallel_2", "mlp": moe,
          "mixer": {"left": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "rot": {"base": 100000.0, "dims": D // 2}},
                    "right": {"heads": z["r_heads"], "dim": z["r_dim"], "vdim": z["r_vdim"]}}}
    p1 = {"type": "parallel", "mlp": moe,
          "mixer": {"left": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "conv": z["conv"], "mask": {"size": s["window"]},
                             "rot": {"base": 1000000.0, "dims": D}},
                    "right": {"heads": z["r_heads"], "kv_heads": z["r_kv"], "dim": z["r_dim"], "vdim": z["r_vdim"], "conv": z["conv"]},
                    "left_scale": 0.5, "right_scale": 0.8}}
    return {"architecture": "Zevedra", "width": s["width"], "vocab": s["vocab"], "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "embedding": {"scale": s["width"] ** 0.5, "bigram": {"buckets": 65521, "mul_prev": 131, "mul_cur": 17}},
            "layers": [p2, p1, dict(p2), dict(p1)], "loop": {"start": 0, "stop": 2, "times": 2}}


def zevedra_products(cfg):
    """((N, K) of the plain dense products, expert weight elements touched, convolution channels) of one token through all six layer runs."""
    W, out, expert, conv = cfg["width"], [], 0, 0
    for li in (0, 1, 0, 1, 2, 3):
        l = cfg["layers"][li]
        a, r = l["mixer"]["left"], l["mixer"]["right"]
        qkv = a["heads"] * a["dim"] + a["kv_heads"] * (a["dim"] + a["vdim"])
        OD, RV = a["heads"] * a["vdim"], r["heads"] * r["vdim"]
        if l["type"] == "parallel":
            RQ = r["kv_heads"] * r["dim"]
            out += [(qkv + a["heads"] + 2 * RQ + 2 * RV + 2 * r["heads"], W), (W, OD + RV)]
            conv += qkv + 2 * RQ + RV
        else:
            out += [(qkv + OD + 2 * r["heads"] * r["dim"] + RV, W), (W, OD), (W, RV)]
        expert += l["mlp"]["router"]["top"] * 3 * l["mlp"]["expert"]["ff"] * W
    return out, expert, conv


def run_zevedra(args, pkg, lib):
    """Zevedra beside Vamidra (attention, short convolution, plain products, norms: the same or like kernels) and beside Mumizen (its
    fixed-decay recurrence is the like kernel of the gated recurrences; its experts) at equal width / head size / expert size and six
    layer runs each: whole-model prompt and decode throughput through the public entry points, device time per kernel category, and for
    every pair of like kernels the distance from its roofline."""
    import numpy as np
    import torch
    hbm, tflops, src = peaks()
    res = {"metric": "Zevedra prompt / decode throughput beside Vamidra and Mumizen at equal size", "impl": "b200", "arch": "Zevedra", "n_gpus": 1,
           "dtype": "bf16", "data": "synthetic random weights", "peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": src}, "sizes": {}}
    rng = np.random.default_rng(0)
    CTX = 1024

    def model(cfg):
        m = pkg.Model.from_config(cfg, dtype="bfloat16", n_ctx=4096, n_seq=16)
        m.synth(0, 7)
        m.finalize()
        return m

    for key in ([args.arch_size] if args.arch_size != "all" else list(SIZES)):
        s, z = SIZES[key], ZEVEDRA_SIZES[key]
        W, V, H, G, D = s["width"], s["vocab"], s["heads"], s["kv_heads"], s["dim"]
        out = {"config": dict(z, width=W, heads=H, kv_heads=G, dim=D, window=s["window"], vocab=V), "layers": 6}
        # ---------------- the new design ----------------
        cfg = zevedra_config(s, z)
        m = model(cfg)
        a = measure(m, V, args, rng, CTX)
        m.close()
        prods, expert, conv_ch = zevedra_products(cfg)
        rec = 6 * z["r_heads"] * z["r_dim"] * z["r_vdim"]          # state entries a token updates, all runs
        for T in (512, 2048):
            pm = a[f"prompt{T}_device_ms"]
            a[f"prompt{T}_dense_frac_of_tensor_peak"] = 2.0 * sum(n * k for n, k in prods) * T / pm["dense"] / 1e9 / tflops
            a[f"prompt{T}_experts_frac_of_tensor_peak"] = 2.0 * expert * T / pm["experts"] / 1e9 / tflops
            vis = 3 * sum(min(i + 1, s["window"]) for i in range(T)) + 3 * T * (T + 1) // 2     # three windowed and three causal runs
            a[f"prompt{T}_attention_tflops"] = 4.0 * D * H * vis / pm["attention"] / 1e9
            a[f"prompt{T}_scan_state_updates_per_ns"] = rec * T / pm["scan"] / 1e6
            a[f"prompt{T}_conv_gbs"] = conv_ch * T * 8.0 / pm["conv"] / 1e6                     # inputs read, outputs written (fp32)
            # three windowed runs: two norms (x read, operand written), both branches' results read in fp32 with the gate and written as operand;
            # three sink runs: a norm, the recurrence's result normed, two products normed and joined onto the stream with the next norm
            OD, RV = H * D, z["r_heads"] * z["r_vdim"]
            a[f"prompt{T}_norm_gbs"] = T * (3 * (12.0 * W + 6.0 * OD + 10.0 * RV) + 3 * (6.0 * W + 6.0 * RV + 18.0 * W)) / pm["norm"] / 1e6
        wb = 2.0 * sum(n * k for n, k in prods)
        a["weight_bytes_per_token"] = wb + 2.0 * expert + 2.0 * V * W
        rows = 3 * min(CTX, s["window"]) + 3 * CTX
        for B in (1, 8):
            pm = a[f"decode_b{B}_device_ms"]
            a[f"decode_b{B}_dense_frac_of_hbm_peak"] = wb / pm["dense"] / 1e6 / hbm
            a[f"decode_b{B}_experts_frac_of_hbm_peak"] = 2.0 * expert * B / pm["experts"] / 1e6 / hbm
            a[f"decode_b{B}_attention_gbs"] = B * rows * G * 2 * D * 4.0 / pm["attention"] / 1e6
            a[f"decode_b{B}_scan_gbs"] = B * rec * 8.0 / pm["scan"] / 1e6                       # the state read and written
            a[f"decode_b{B}_whole_step_frac_of_hbm_peak"] = a["weight_bytes_per_token"] / a[f"decode_b{B}_ms_per_step"] / 1e6 / hbm
        out["zevedra"] = a
        # ---------------- Vamidra: windowed attention, convolution + scan, plain products, norms ----------------
        vcfg = vamidra_config(s)
        m = model(vcfg)
        b = measure(m, V, args, rng, CTX)
        m.close()
        shapes = dense_shapes(s, vcfg)
        vconv = 3 * (s["ssm_heads"] * s["vdim"] + 2 * s["groups"] * s["state"])
        vrec = 3 * s["ssm_heads"] * s["state"] * s["vdim"]
        for T in (512, 2048):
            pm = b[f"prompt{T}_device_ms"]
            b[f"prompt{T}_dense_frac_of_tensor_peak"] = 2.0 * sum(n * k for n, k in shapes) * T / pm["dense"] / 1e9 / tflops
            vis = sum(min(i + 1, s["window"]) + max(0, min(s["keep_first"], i + 1 - s["window"])) for i in range(T))
            b[f"prompt{T}_attention_tflops"] = 3 * 4.0 * D * H * vis / pm["attention"] / 1e9
            b[f"prompt{T}_scan_state_updates_per_ns"] = vrec * T / pm["scan"] / 1e6
            b[f"prompt{T}_conv_gbs"] = vconv * T * 8.0 / pm["conv"] / 1e6
            b[f"prompt{T}_norm_gbs"] = (12 * T * W * 6.0 + 3 * T * s["ssm_heads"] * s["vdim"] * 10.0) / pm["norm"] / 1e6
        wbv = 2.0 * sum(n * k for n, k in shapes)
        b["weight_bytes_per_token"] = wbv + 2.0 * V * W
        vrows = min(CTX, s["window"] + s["keep_first"])
        for B in (1, 8):
            pm = b[f"decode_b{B}_device_ms"]
            b[f"decode_b{B}_dense_frac_of_hbm_peak"] = wbv / pm["dense"] / 1e6 / hbm
            b[f"decode_b{B}_attention_gbs"] = 3 * B * vrows * G * 2 * D * 4.0 / pm["attention"] / 1e6
            b[f"decode_b{B}_scan_gbs"] = B * vrec * 8.0 / pm["scan"] / 1e6
            b[f"decode_b{B}_whole_step_frac_of_hbm_peak"] = b["weight_bytes_per_token"] / b[f"decode_b{B}_ms_per_step"] / 1e6 / hbm
        out["vamidra"] = b
        # ---------------- Mumizen: the fixed-decay recurrence and the experts at equal sizes ----------------
        mz = dict(MUMIZEN_SIZES[key], experts=z["experts"], top=z["top"], expert_ff=z["expert_ff"])
        mcfg = mumizen_config(s, mz)
        m = model(mcfg)
        c = measure(m, V, args, rng, CTX)
        m.close()
        _, mexpert = mumizen_products(mcfg, True)
        n_lin = sum(l["type"] != "latent_attention" for l in mcfg["layers"])
        mrec = n_lin * mz["heads"] * mz["dim"] * mz["vdim"]
        e = {}
        for T in (512, 2048):
            pm = c[f"prompt{T}_device_ms"]
            e[f"prompt{T}_experts_frac_of_tensor_peak"] = 2.0 * mexpert * T / pm["experts"] / 1e9 / tflops
            e[f"prompt{T}_scan_state_updates_per_ns"] = mrec * T / pm["scan"] / 1e6
        for B in (1, 8):
            pm = c[f"decode_b{B}_device_ms"]
            e[f"decode_b{B}_experts_frac_of_hbm_peak"] = 2.0 * mexpert * B / pm["experts"] / 1e6 / hbm
            e[f"decode_b{B}_scan_gbs"] = B * mrec * 8.0 / pm["scan"] / 1e6
        out["mumizen_like_kernels"] = e
        res["sizes"][key] = out
        torch.cuda.empty_cache()
    res["gpu_launches"] = int(lib.c.pb200_kernel_launches())
    print(json.dumps(res))
    return res
