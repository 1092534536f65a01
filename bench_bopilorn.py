"""``bench.py --arch bopilorn``: the Bopilorn architecture at layer sizes that resemble real models,
beside Qwen2 (the engine's closest model) at equal width, depth, heads and ACTIVE feed-forward size
(Qwen2's dense inner width = chosen experts x an expert's inner width).

Per size: a 2,048-token prefill and decode steps at batch 8 around a context of 2,048 tokens, both
models with random weights in bfloat16, timed on the device (CUDA events, median of the regions;
weights and caches together exceed the L2).  Then each kernel that Bopilorn adds, alone, with the
bytes or flops it must move and the fraction of the measured roofline that makes, next to the like
kernel of Qwen2 where there is one.  One JSON line.
"""

from __future__ import annotations

import json
import sys

import bench_zazasun as common
from bench_zazasun import PREFILL, Bench, _segments, _time, model_points

SIZES = {
    # width, heads, experts, chosen experts, an expert's inner width, groups (count, kept), layers, vocabulary
    "896": dict(width=896, layers=12, vocab=32000, heads=14, kv_heads=2, dim=64, experts=16, top=2, ff=2432, groups=(4, 2)),
    "2048": dict(width=2048, layers=12, vocab=32000, heads=16, kv_heads=4, dim=128, experts=64, top=6, ff=1408, groups=(8, 4)),
    "4096": dict(width=4096, layers=8, vocab=32000, heads=32, kv_heads=8, dim=128, experts=32, top=4, ff=2048, groups=(4, 2)),
}


def bopilorn_config(size):
    from mini_llm_runtime_b200.config import config_from_dict

    s = SIZES[size]
    mixer = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5,
             "rot": {"base": 10000.0, "dims": s["dim"], "scaling": {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0}}}
    mlp = {"kind": "moe", "expert": {"ff": s["ff"]},
           "router": {"experts": s["experts"], "top": s["top"], "groups": {"count": s["groups"][0], "keep": s["groups"][1]}}}
    return config_from_dict({"architecture": "Bopilorn", "vocab": s["vocab"], "width": s["width"],
                             "max_positions": common.MAX_POSITIONS, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
                             "layers": [{"type": "attention", "mixer": mixer, "mlp": mlp}] * s["layers"]})


def qwen_config(size):
    from mini_llm_runtime_b200.config import Qwen2Config

    s = SIZES[size]
    return Qwen2Config(vocab_size=s["vocab"], hidden_size=s["width"], intermediate_size=s["top"] * s["ff"],
                       num_hidden_layers=s["layers"], num_attention_heads=s["heads"],
                       num_key_value_heads=s["kv_heads"], head_dim=s["dim"],
                       max_position_embeddings=common.MAX_POSITIONS, rms_norm_eps=1e-6, rope_theta=1e6,
                       hidden_act="silu", tie_word_embeddings=False)


def experts_touched(experts, top, rows):
    """Expected number of distinct experts that `rows` rows with `top` choices each read (uniform router)."""
    return experts * (1.0 - (1.0 - top / experts) ** rows)


def bopilorn_numbers(size, batch=8):
    """Bytes a decode step of `batch` rows must read and flops of a prefill, from the sizes."""
    s = SIZES[size]
    width, layers = s["width"], s["layers"]
    attention = (s["heads"] + 2 * s["kv_heads"]) * s["dim"] * width + width * s["heads"] * s["dim"]
    expert = 3 * width * s["ff"]
    router = s["experts"] * width
    read = attention + 2 * router + experts_touched(s["experts"], s["top"], batch) * expert     # the router is 32-bit
    active = attention + router + s["top"] * expert
    head = s["vocab"] * width
    return {"weight_bytes": int(2 * (layers * read + head)),
            "kv_bytes_per_token": 2 * layers * s["kv_heads"] * s["dim"] * 2,
            "linear_flops_per_token": 2 * layers * active, "head_flops_per_row": 2 * head,
            "attention_flops": lambda rows, before=0: layers * 4 * s["heads"] * s["dim"] * (rows * before + rows * (rows + 1) // 2)}


def prefill_weight_bytes(size):
    """Bytes of weights a prefill of 2,048 rows reads: every expert of every layer once."""
    s = SIZES[size]
    width = s["width"]
    attention = (s["heads"] + 2 * s["kv_heads"]) * s["dim"] * width + width * s["heads"] * s["dim"]
    return int(2 * (s["layers"] * (attention + 2 * s["experts"] * width + s["experts"] * 3 * width * s["ff"])
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
    width, heads, kv_heads, dim, experts, top, ff = (s["width"], s["heads"], s["kv_heads"], s["dim"], s["experts"], s["top"],
                                                      s["ff"])
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

    rope = build_part("position", PartSpec("rope_pairs", {"head_dim": dim, "theta": 10000.0, "layout": "interleaved",
                                                           "scaling": {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0}}), bf16)
    value_rope = build_part("position", PartSpec("rope_pairs", {"head_dim": dim, "theta": 10000.0, "layout": "interleaved"}), bf16)
    half_rope = build_part("position", PartSpec("rope_half", {"head_dim": dim, "theta": 1e6}), bf16)
    for part in (rope, value_rope, half_rope):
        part.load({}, torch.device("cuda"))
    # the experts' matrices and the dense matrices of the same active size
    gate_up = (torch.randn(experts, 2 * ff, width, device="cuda") * 0.02).to(bf16)
    down = (torch.randn(experts, width, ff, device="cuda") * 0.02).to(bf16)
    dense_gate_up = (torch.randn(2 * top * ff, width, device="cuda") * 0.02).to(bf16)
    dense_down = (torch.randn(width, top * ff, device="cuda") * 0.02).to(bf16)
    router = torch.randn(experts, width, device="cuda") * 0.05
    correction = torch.randn(experts, device="cuda") * 0.01

    cases = {"prefill": _segments([PREFILL], [0]), "decode": _segments([1] * 8, [2047] * 8)}
    for label, ctx in cases.items():
        rows = int(ctx.lengths.sum())
        page, context = 16, int(ctx.positions.max() + ctx.lengths.max())
        pages_per_request = -(-context // page)
        table = torch.arange(ctx.num_segments * pages_per_request, dtype=torch.int32, device="cuda").view(ctx.num_segments, -1)
        k_pool = torch.randn(ctx.num_segments * pages_per_request, kv_heads, page, dim, device="cuda").to(bf16)
        v_pool = torch.randn_like(k_pool)
        positions = torch.cat([torch.arange(int(p), int(p) + int(n), dtype=torch.int32)
                               for p, n in zip(ctx.positions, ctx.lengths)]).cuda()
        slots = torch.cat([torch.arange(int(p), int(p) + int(n), dtype=torch.int64) + i * pages_per_request * page
                           for i, (p, n) in enumerate(zip(ctx.positions, ctx.lengths))]).cuda()
        qkv_width = (heads + 2 * kv_heads) * dim
        qkv32 = torch.randn(rows, qkv_width, device="cuda")
        q_weight, k_weight = torch.ones(heads * dim, device="cuda"), torch.ones(kv_heads * dim, device="cuda")
        record(f"rotated_prepare.{label}",
               _time(lambda: k.rotated_prepare(qkv32, positions, q_weight, k_weight, 1e-6, rope.rotary_frequencies(),
                                               rope.magnitude, value_rope.rotary_frequencies(), True, True, slots, k_pool,
                                               v_pool, heads, kv_heads, dim, dim), flush),
               rows * qkv_width * 6)
        qkv16 = qkv32.to(bf16)
        record(f"qwen.rope_kv_write.{label}",
               _time(lambda: k.rope_kv_write(qkv16, positions, half_rope.rotary_frequencies(), slots, k_pool, v_pool, heads,
                                             kv_heads, dim, True), flush),
               rows * qkv_width * 4)
        # attention over a paged cache that already holds every position: the kernel is Qwen2's; the
        # way back of the values' rotation follows it
        arrays, counts = plan_attention(ctx.lengths, ctx.positions)
        arrays = {name: torch.from_numpy(value).cuda() for name, value in arrays.items()}
        batch = AttentionBatch(ctx.seg_q_start, ctx.seg_q_len, ctx.seg_pos0, ctx.seg_slot, table, ctx.num_segments,
                               ctx.max_q_len, context, arrays, counts)
        q = (torch.randn(rows, heads * dim, device="cuda") * 0.2).to(bf16)
        pairs = sum(int(p) + i + 1 for p, n in zip(ctx.positions, ctx.lengths) for i in range(int(n)))
        attention_bytes = context * ctx.num_segments * kv_heads * dim * 4 + 2 * rows * heads * dim * 2
        record(f"attention.{label}",
               _time(lambda: k.paged_attention(q, k_pool, v_pool, batch, heads, kv_heads, dim, dim ** -0.5, None), flush),
               attention_bytes, pairs * heads * 4 * dim)
        mixed = torch.randn(rows, heads * dim, device="cuda").to(bf16)
        record(f"turn_heads.{label}",
               _time(lambda: k.turn_heads(mixed, positions, value_rope.rotary_frequencies(), heads, dim, True, -1.0), flush),
               rows * heads * dim * 4)
        # router, and the experts beside the dense feed-forward of the same active size
        h = torch.randn(rows, width, device="cuda").to(bf16)
        record(f"route_experts.{label}",
               _time(lambda: k.route_experts(h, router, correction, top, s["groups"][0], s["groups"][1]), flush),
               rows * width * 2 + experts * width * 4, 2 * rows * experts * width)
        chosen, weights = k.route_experts(h, router, correction, top, s["groups"][0], s["groups"][1])
        flops = 2 * rows * top * 3 * ff * width
        touched = experts if rows > experts else experts_touched(experts, top, rows)
        expert_bytes = touched * 3 * ff * width * 2 + rows * width * 6
        record(f"routed_experts.{label}", _time(lambda: k.routed_experts(h, chosen, weights, gate_up, down, 64), flush),
               expert_bytes, flops)
        record(f"qwen.feed_forward.{label}",
               _time(lambda: k.linear(k.linear_swiglu(h, dense_gate_up, 64), dense_down), flush),
               3 * top * ff * width * 2 + rows * width * 4, flops)
        x = torch.randn(rows, width, device="cuda", dtype=f32)
        delta = torch.randn(rows, width, device="cuda", dtype=f32)
        vector = lambda: torch.randn(width, device="cuda")      # noqa: E731
        zero = torch.zeros(width, device="cuda")
        pair, post = (vector(), zero), (vector(), zero)
        record(f"add_layer_norm_layer_norm.{label}",
               _time(lambda: k.layer_norm_step(x, 1e-6, delta=delta, delta_norm=post, norm=pair, out_dtype=bf16), flush),
               rows * width * 14)
        xb, db = x.to(bf16), delta.to(bf16)
        record(f"qwen.add_rms_norm.{label}", _time(lambda: k.add_rms_norm(xb, db, None, 1e-6), flush), rows * width * 8)
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
    record = {"metric": "Bopilorn beside Qwen2 at equal active sizes: prefill of 2,048 tokens and decode at batch 8",
              "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)", "n_gpus": 1,
              "context": 2048, "peaks": peak, "sizes": {}, "kernels": {}}
    with host.ClockSampler() as clocks:
        for size in SIZES:
            entry = {}
            for name, make in (("bopilorn", bopilorn_config), ("qwen2", qwen_config)):
                config = make(size)
                if name == "bopilorn":
                    numbers = bopilorn_numbers(size)
                else:
                    numbers = host.model_numbers(config, config.num_hidden_layers)
                bench = Bench(f"{name} {size}", config, numbers, host)
                entry[name] = model_points(bench, host, args, peak)
                entry[name]["layers"] = len(bench.model.blocks)
                # the prefill's roofline: the slower of its flops at the measured peak and the bytes it
                # must read (every weight once: 2,048 rows touch every expert) at the measured bandwidth
                flops = entry[name]["prefill_frac_of_bf16_peak"] * peak["bf16_tflops"] * 1e12 * entry[name]["prefill_2048_ms"] / 1e3
                weights = prefill_weight_bytes(size) if name == "bopilorn" else numbers["weight_bytes"]
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
