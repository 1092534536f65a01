"""``bench.py --arch ratilorn``: the Ratilorn architecture at layer sizes that resemble real models,
beside Bopilorn (the engine's closest model: routed experts, a 32-bit stream, an attention whose q, k
and v are prepared by a kernel of its own) at equal width, depth, heads and experts.

Per size: a 2,048-token prefill and decode steps at batch 8 around a context of 2,048 tokens, both
models with random weights in bfloat16, timed on the device (CUDA events, median of the regions;
weights and caches together exceed the L2).  Then each kernel that Ratilorn adds, alone, with the
bytes or flops it must move and the fraction of the measured roofline that makes, next to the like
kernel of an existing model where there is one.  One JSON line.
"""

from __future__ import annotations

import json
import sys

import bench_bopilorn
import bench_zazasun as common
from bench_zazasun import PREFILL, Bench, _segments, _time, model_points

SIZES = {
    # groups of (parallel, parallel, attention) layers; the state-space branch as wide as the model
    "896": dict(width=896, groups=4, vocab=32000, heads=14, kv_heads=2, dim=64, ssm=dict(heads=14, vdim=64, state=64),
                experts=16, top=2, ff=2432, router_groups=(4, 2), shared=2432),
    "2048": dict(width=2048, groups=4, vocab=32000, heads=16, kv_heads=4, dim=128, ssm=dict(heads=32, vdim=64, state=128),
                 experts=64, top=6, ff=1408, router_groups=(8, 4), shared=1408),
}
TAPS = 4


def ratilorn_config(size):
    from mini_llm_runtime_b200.config import config_from_dict

    s = SIZES[size]
    heads = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5}
    right = {**s["ssm"], "groups": 1, "conv": TAPS, "norm_groups": 1}
    mlp = {"kind": "moe", "expert": {"ff": s["ff"]}, "shared": {"ff": s["shared"]},
           "router": {"experts": s["experts"], "top": s["top"],
                      "groups": {"count": s["router_groups"][0], "keep": s["router_groups"][1]}}}
    group = [{"type": "parallel", "mixer": {"left": heads, "right": right}, "mlp": mlp},
             {"type": "parallel", "mixer": {"left": heads, "right": right}, "mlp": mlp},
             {"type": "attention", "mixer": {**heads, "v_mix": True}, "mlp": mlp}]
    return config_from_dict({"architecture": "Ratilorn", "vocab": s["vocab"], "width": s["width"],
                             "max_positions": common.MAX_POSITIONS, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
                             "layers": group * s["groups"]})


def bopilorn_config(size):
    from mini_llm_runtime_b200.config import config_from_dict

    s = SIZES[size]
    mixer = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5,
             "rot": {"base": 10000.0, "dims": s["dim"]}}
    mlp = {"kind": "moe", "expert": {"ff": s["ff"]},
           "router": {"experts": s["experts"], "top": s["top"],
                      "groups": {"count": s["router_groups"][0], "keep": s["router_groups"][1]}}}
    return config_from_dict({"architecture": "Bopilorn", "vocab": s["vocab"], "width": s["width"],
                             "max_positions": common.MAX_POSITIONS, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
                             "layers": [{"type": "attention", "mixer": mixer, "mlp": mlp}] * (3 * s["groups"])})


def _pieces(size):
    s = SIZES[size]
    width = s["width"]
    attention = (s["heads"] + 2 * s["kv_heads"]) * s["dim"] * width + width * s["heads"] * s["dim"]
    inner = s["ssm"]["heads"] * s["ssm"]["vdim"]
    state_space = (2 * inner + 2 * s["ssm"]["state"] + s["ssm"]["heads"]) * width + width * inner
    return s, width, attention, state_space, 3 * width * s["ff"], 3 * width * s["shared"], s["experts"] * width


def ratilorn_numbers(size, batch=8):
    """Bytes a decode step of `batch` rows must read and flops of a prefill, from the sizes."""
    s, width, attention, state_space, expert, shared, router = _pieces(size)
    layers = 3 * s["groups"]
    parallel_layers = 2 * s["groups"]
    touched = bench_bopilorn.experts_touched(s["experts"], s["top"], batch)
    read = layers * (attention + 2 * router + touched * expert + shared) + parallel_layers * state_space
    active = layers * (attention + router + s["top"] * expert + shared) + parallel_layers * state_space
    head = s["vocab"] * width
    ssm = s["ssm"]
    state_bytes = parallel_layers * 2 * 4 * ssm["heads"] * ssm["vdim"] * ssm["state"]

    def sequence_flops(rows, before=0):
        pairs = rows * before + rows * (rows + 1) // 2
        scores = layers * pairs * s["heads"] * 4 * s["dim"]
        mixing = s["groups"] * pairs * s["heads"] * s["heads"] * 2
        scan = parallel_layers * rows * ssm["heads"] * ssm["vdim"] * ssm["state"] * 4
        return scores + mixing + scan

    return {"weight_bytes": int(2 * (read + head)), "kv_bytes_per_token": 2 * layers * s["kv_heads"] * s["dim"] * 2,
            "cache_bytes_per_request": state_bytes, "linear_flops_per_token": 2 * active, "head_flops_per_row": 2 * head,
            "attention_flops": sequence_flops}


def prefill_weight_bytes(size):
    s, width, attention, state_space, expert, shared, router = _pieces(size)
    layers = 3 * s["groups"]
    return int(2 * (layers * (attention + 2 * router + s["experts"] * expert + shared) + 2 * s["groups"] * state_space
                    + s["vocab"] * width))


def kernel_points(size, peak):
    """Each new kernel alone: 2,048 rows of one request (prefill) and 8 requests of one row (decode)."""
    import torch

    from mini_llm_runtime_b200 import ops
    from mini_llm_runtime_b200.config import PartSpec
    from mini_llm_runtime_b200.ops.cuda_ops import AttentionBatch, plan_attention
    from mini_llm_runtime_b200.parts import build_part

    k = ops.current()
    s = SIZES[size]
    width, heads, kv_heads, dim = s["width"], s["heads"], s["kv_heads"], s["dim"]
    ssm = s["ssm"]
    inner, n = ssm["heads"] * ssm["vdim"], ssm["state"]
    channels = inner + 2 * n
    flush = torch.zeros(96 << 20, dtype=torch.float32, device="cuda")      # 384 MB, three times the L2
    bf16, f32 = torch.bfloat16, torch.float32
    hbm = peak["hbm_gbs"] * 1e9
    out = {}

    def record(name, micros, nbytes=None, flops=None):
        entry = {"us": round(micros, 2)}
        if nbytes is not None:
            entry["bytes"] = int(nbytes)
            entry["hbm_frac"] = round(nbytes / (micros * 1e-6) / hbm, 4) if micros > 0 else None
        if flops is not None:
            entry["tflops"] = round(flops / (micros * 1e-6) / 1e12, 3) if micros > 0 else None
            entry["bf16_peak_frac"] = round(flops / (micros * 1e-6) / (peak["bf16_tflops"] * 1e12), 5) if micros > 0 else None
        out[name] = entry

    rope = build_part("position", PartSpec("rope_pairs", {"head_dim": dim, "theta": 10000.0, "layout": "interleaved"}), bf16)
    rope.load({}, torch.device("cuda"))
    vector = lambda size_: torch.randn(size_, device="cuda")      # noqa: E731
    cases = {"prefill": _segments([PREFILL], [0]), "decode": _segments([1] * 8, [2047] * 8)}
    for label, ctx in cases.items():
        rows = int(ctx.lengths.sum())
        page, context = 16, int(ctx.positions.max() + ctx.lengths.max())
        pages_per_request = -(-context // page)
        table = torch.arange(ctx.num_segments * pages_per_request, dtype=torch.int32, device="cuda").view(ctx.num_segments, -1)
        k_pool = torch.randn(ctx.num_segments * pages_per_request, kv_heads, page, dim, device="cuda").to(bf16)
        v_pool = torch.randn_like(k_pool)
        positions = torch.cat([torch.arange(int(p), int(p) + int(c), dtype=torch.int32)
                               for p, c in zip(ctx.positions, ctx.lengths)]).cuda()
        slots = torch.cat([torch.arange(int(p), int(p) + int(c), dtype=torch.int64) + i * pages_per_request * page
                           for i, (p, c) in enumerate(zip(ctx.positions, ctx.lengths))]).cuda()
        qkv_width = (heads + 2 * kv_heads) * dim
        qkv32 = torch.randn(rows, qkv_width, device="cuda")
        other = torch.randn(rows, qkv_width, device="cuda")[:, (heads + kv_heads) * dim:]
        mix = torch.full((1,), 0.5, device="cuda")
        head_weight = torch.ones(dim, device="cuda")
        record(f"head_norm_kv_write.{label}",
               _time(lambda: k.head_norm_kv_write(qkv32, head_weight, head_weight, 1e-6, slots, k_pool, v_pool, heads, kv_heads,
                                                  dim, dim, True, other_values=other, mix=mix), flush),
               rows * qkv_width * 6 + rows * kv_heads * dim * 4)
        q_weight, k_weight = torch.ones(heads * dim, device="cuda"), torch.ones(kv_heads * dim, device="cuda")
        record(f"bopilorn.rotated_prepare.{label}",
               _time(lambda: k.rotated_prepare(qkv32, positions, q_weight, k_weight, 1e-6, rope.rotary_frequencies(),
                                               rope.magnitude, rope.rotary_frequencies(), True, True, slots, k_pool, v_pool,
                                               heads, kv_heads, dim, dim), flush),
               rows * qkv_width * 6)
        arrays, counts = plan_attention(ctx.lengths, ctx.positions)
        arrays = {name: torch.from_numpy(value).cuda() for name, value in arrays.items()}
        batch = AttentionBatch(ctx.seg_q_start, ctx.seg_q_len, ctx.seg_pos0, ctx.seg_slot, table, ctx.num_segments,
                               ctx.max_q_len, context, arrays, counts)
        q = (torch.randn(rows, heads * dim, device="cuda") * 0.2).to(bf16)
        pairs = sum(int(p) + i + 1 for p, c in zip(ctx.positions, ctx.lengths) for i in range(int(c)))
        attention_bytes = context * ctx.num_segments * kv_heads * dim * 4 + 2 * rows * heads * dim * 2
        r1, r2, pb = torch.rand(heads, device="cuda"), torch.rand(heads, device="cuda"), vector(heads)
        talk = torch.eye(heads, device="cuda") + 0.1 * torch.randn(heads, heads, device="cuda")
        record(f"sigmoid_attention.{label}",
               _time(lambda: k.sigmoid_attention(q, k_pool, v_pool, batch, heads, kv_heads, dim, dim, dim ** -0.5,
                                                 distance=(r1, r2), score_bias=pb, head_mix=talk), flush),
               attention_bytes, pairs * heads * (4 * dim + 2 * heads))
        record(f"softmax_attention.{label}",
               _time(lambda: k.paged_attention(q, k_pool, v_pool, batch, heads, kv_heads, dim, dim ** -0.5, None), flush),
               attention_bytes, pairs * heads * 4 * dim)
        # the state-space branch: convolution, recurrence, gated norm; beside the forget-gate recurrence
        projected = torch.randn(rows, 2 * inner + 2 * n + ssm["heads"], device="cuda") * 0.5
        conv, conv_bias = torch.randn(channels, TAPS, device="cuda") * 0.3, vector(channels) * 0.1
        conv_state = torch.zeros(8, TAPS - 1, channels, device="cuda")
        record(f"causal_conv.{label}",
               _time(lambda: k.causal_conv(projected[:, inner:inner + channels], conv, conv_bias, conv_state, ctx), flush),
               rows * channels * 8 + (2 * ctx.num_segments * (TAPS - 1) * channels * 4 if label == "decode" else 0))
        mixed = k.causal_conv(projected[:, inner:inner + channels], conv, conv_bias, conv_state, ctx)
        dt_bias, a_log, skip = vector(ssm["heads"]) * 0.1, -torch.rand(ssm["heads"], device="cuda"), vector(ssm["heads"])
        state = torch.zeros(8, ssm["heads"], ssm["vdim"], n, device="cuda")
        scan_bytes = rows * (inner * 8 + 2 * n * 4 + ssm["heads"] * 4) + 2 * ctx.num_segments * inner * n * 4
        record(f"state_space_scan.{label}",
               _time(lambda: k.state_space_scan(mixed[:, :inner], mixed[:, inner:inner + n], mixed[:, inner + n:],
                                                projected[:, inner + channels:], dt_bias, a_log, skip, state, ctx,
                                                ssm["heads"], ssm["vdim"], n, 1), flush),
               scan_bytes, rows * inner * n * 4)
        keys = ssm["heads"] * n
        fq, ff_ = (torch.randn(rows, keys, device="cuda") * 0.3 for _ in range(2))
        fv = torch.randn(rows, inner, device="cuda") * 0.3
        fstate = torch.zeros(8, ssm["heads"], n, ssm["vdim"], device="cuda")
        record(f"zazasun.forget_gate_recurrence.{label}",
               _time(lambda: k.forget_gate_recurrence(fq, ff_, fv, vector(keys) * 0.1, torch.rand(keys, device="cuda"),
                                                      torch.ones(ssm["vdim"], device="cuda"), 1e-6, fstate, ctx, ssm["heads"],
                                                      n, ssm["vdim"], bf16), flush),
               rows * (2 * keys * 4 + inner * 6) + 2 * ctx.num_segments * inner * n * 4, rows * inner * n * 4)
        y, norm_weight = torch.randn(rows, inner, device="cuda"), torch.ones(inner, device="cuda")
        record(f"gated_group_norm.{label}",
               _time(lambda: k.gated_group_norm(y, projected[:, :inner], norm_weight, 1e-6, 1, bf16), flush), rows * inner * 10)
        # the stream: x += norm(delta) with the rows out in 16 bits; the two branches' mean
        x, delta = torch.randn(rows, width, device="cuda"), torch.randn(rows, width, device="cuda")
        w1, w2 = torch.ones(width, device="cuda"), torch.ones(width, device="cuda")
        record(f"rms_norm_step.{label}",
               _time(lambda: k.rms_norm_step(x, 1e-6, delta=delta, delta_weight=w1, out_dtype=bf16), flush), rows * width * 14)
        zero = torch.zeros(width, device="cuda")
        record(f"bopilorn.layer_norm_step.{label}",
               _time(lambda: k.layer_norm_step(x, 1e-6, delta=delta, delta_norm=(w1, zero), norm=(w2, zero), out_dtype=bf16),
                     flush), rows * width * 14)
        record(f"normed_mean.{label}", _time(lambda: k.normed_mean(x, w1, delta, w2, 1e-6, 0.5), flush), rows * width * 12)
        del k_pool, v_pool
        torch.cuda.empty_cache()
    k.raise_if_device_error()
    return out


def run(args, host):
    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    peak = host.peaks()
    record = {"metric": "Ratilorn beside Bopilorn at equal sizes: prefill of 2,048 tokens and decode at batch 8",
              "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)", "n_gpus": 1,
              "context": 2048, "peaks": peak, "sizes": {}, "kernels": {}}
    with host.ClockSampler() as clocks:
        for size in SIZES:
            entry = {}
            for name, make in (("ratilorn", ratilorn_config), ("bopilorn", bopilorn_config)):
                config = make(size)
                if name == "ratilorn":
                    numbers, weights = ratilorn_numbers(size), prefill_weight_bytes(size)
                else:
                    bench_bopilorn.SIZES[size + "r"] = dict(
                        width=SIZES[size]["width"], layers=3 * SIZES[size]["groups"], vocab=SIZES[size]["vocab"],
                        heads=SIZES[size]["heads"], kv_heads=SIZES[size]["kv_heads"], dim=SIZES[size]["dim"],
                        experts=SIZES[size]["experts"], top=SIZES[size]["top"], ff=SIZES[size]["ff"],
                        groups=SIZES[size]["router_groups"])
                    numbers = bench_bopilorn.bopilorn_numbers(size + "r")
                    weights = bench_bopilorn.prefill_weight_bytes(size + "r")
                bench = Bench(f"{name} {size}", config, numbers, host)
                entry[name] = model_points(bench, host, args, peak)
                entry[name]["layers"] = len(bench.model.blocks)
                flops = entry[name]["prefill_frac_of_bf16_peak"] * peak["bf16_tflops"] * 1e12 * entry[name]["prefill_2048_ms"] / 1e3
                bound_ms = max(flops / (peak["bf16_tflops"] * 1e12), weights / (peak["hbm_gbs"] * 1e9)) * 1e3
                entry[name]["prefill_roofline_ms"] = round(bound_ms, 3)
                entry[name]["prefill_frac_of_roofline"] = round(bound_ms / entry[name]["prefill_2048_ms"], 4)
                bench.close()
            record["sizes"][size] = entry
            record["kernels"][size] = kernel_points(size, peak)
            print(f"[bench] {size}: {json.dumps(entry)}", file=sys.stderr)
            print(f"[bench] {size} kernels: {json.dumps(record['kernels'][size])}", file=sys.stderr)
    record["clocks"] = clocks.summary()
    print(json.dumps(record))
    return 0
