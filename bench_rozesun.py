"""``bench.py --arch rozesun``: the Rozesun architecture at layer sizes that resemble real models,
beside Qwen2 (the engine's closest model) at equal width, depth and feed-forward size.

Per size: a 2,048-token prefill and decode steps at batch 8 around a context of 2,048 tokens, both
models with random weights in bfloat16, timed on the device (CUDA events, median of the regions;
weights and caches together exceed the L2).  Then each kernel that Rozesun adds, alone, with the
bytes or flops it must move and the fraction of the measured roofline that makes, next to the like
kernel of Qwen2 where there is one.  One JSON line.
"""

from __future__ import annotations

import json
import math
import sys

import bench_zazasun as common
from bench_zazasun import PREFILL, Bench, _segments, _time, model_points

SIZES = {
    # width, feed-forward, groups of (windowed, full, full) layers, vocabulary; latent sizes in the
    # proportions of published latent-attention models (latent 4 x a head's size, turned part half a head)
    "896": dict(width=896, ff=4864, groups=4, vocab=32000,
                mixer=dict(heads=14, dim=64, rot_dim=32, vdim=64, kv_rank=256, q_rank=384),
                qwen=dict(heads=14, kv_heads=2, head_dim=64)),
    "2048": dict(width=2048, ff=8192, groups=4, vocab=32000,
                 mixer=dict(heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=768),
                 qwen=dict(heads=16, kv_heads=4, head_dim=128)),
}
WINDOW = 1024
LIMIT = 7.0


def rozesun_config(size):
    from mini_llm_runtime_b200.config import config_from_dict

    s = SIZES[size]
    mlp = {"kind": "dense", "ff": s["ff"], "limit": LIMIT}
    a = s["mixer"]
    mixer = dict(a, rot={"base": 10000.0, "dims": a["rot_dim"]}, scale=1.0 / math.sqrt(a["dim"] + a["rot_dim"]))
    group = [{"type": "latent_attention_2", "mixer": dict(mixer, mask={"size": WINDOW}), "mlp": mlp},
             {"type": "latent_attention", "mixer": mixer, "mlp": mlp},
             {"type": "latent_attention", "mixer": mixer, "mlp": mlp}]
    return config_from_dict({"architecture": "Rozesun", "vocab": s["vocab"], "width": s["width"],
                             "max_positions": common.MAX_POSITIONS, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
                             "layers": group * s["groups"]})


def qwen_config(size):
    from mini_llm_runtime_b200.config import Qwen2Config

    s = SIZES[size]
    return Qwen2Config(vocab_size=s["vocab"], hidden_size=s["width"], intermediate_size=s["ff"],
                       num_hidden_layers=3 * s["groups"], num_attention_heads=s["qwen"]["heads"],
                       num_key_value_heads=s["qwen"]["kv_heads"], head_dim=s["qwen"]["head_dim"],
                       max_position_embeddings=common.MAX_POSITIONS, rms_norm_eps=1e-6, rope_theta=1e6,
                       hidden_act="silu", tie_word_embeddings=False)


def rozesun_numbers(config, context):
    """Bytes a decode step must read and flops of a prefill, from the configuration."""
    width = config.width
    matrices = 0
    cache_bytes = 0
    terms = []
    for layer in config.layers:
        a = layer.mixer_args
        gate = a["heads"] if layer.type == "latent_attention_2" else a["heads"] * a["vdim"]
        matrices += (a["q_rank"] + a["kv_rank"] + a["rot_dim"] + gate) * width
        matrices += a["heads"] * (a["dim"] + a["rot_dim"]) * a["q_rank"]
        matrices += a["heads"] * (a["dim"] + a["vdim"]) * a["kv_rank"] + width * a["heads"] * a["vdim"]
        matrices += 3 * width * layer.ff
        keys = min(context, a["window"]) if a["window"] else context
        cache_bytes += keys * (a["kv_rank"] + a["rot_dim"]) * 2
        terms.append(a)

    def sequence_flops(rows):
        total = 0
        for a in terms:
            pairs = sum(min(p + 1, a["window"]) if a["window"] else p + 1 for p in range(rows))
            total += pairs * a["heads"] * 2 * (2 * a["kv_rank"] + a["rot_dim"])
        return total

    head = config.vocab * width
    return {"weight_bytes": 2 * (matrices + head), "kv_bytes_per_token": 0, "cache_bytes_per_request": cache_bytes,
            "linear_flops_per_token": 2 * matrices, "head_flops_per_row": 2 * head,
            "attention_flops": lambda rows, before=0: sequence_flops(rows)}


def kernel_points(size, peak):
    """Each new kernel alone: 2,048 rows of one request (prefill) and 8 requests of one row (decode)."""
    import torch

    from mini_llm_runtime_b200 import ops
    from mini_llm_runtime_b200.ops.cuda_ops import AttentionBatch, plan_attention

    k = ops.current()
    s = SIZES[size]
    a = s["mixer"]
    width, heads, dim, rot, vdim, rank, q_rank = (s["width"], a["heads"], a["dim"], a["rot_dim"], a["vdim"], a["kv_rank"],
                                                  a["q_rank"])
    flush = torch.zeros(96 << 20, dtype=torch.float32, device="cuda")      # 384 MB, three times the L2
    bf16, f32 = torch.bfloat16, torch.float32
    hbm = peak["hbm_gbs"] * 1e9
    out = {}

    def record(name, micros, nbytes=None, flops=None):
        entry = {"us": round(micros, 2)}
        if nbytes is not None:
            entry["bytes"] = int(nbytes)
            entry["hbm_frac"] = round(nbytes / (micros * 1e-6) / hbm, 4)
        if flops is not None:
            entry["tflops"] = round(flops / (micros * 1e-6) / 1e12, 3)
            entry["bf16_peak_frac"] = round(flops / (micros * 1e-6) / (peak["bf16_tflops"] * 1e12), 5)
        out[name] = entry

    cases = {"prefill": _segments([PREFILL], [0]), "decode": _segments([1] * 8, [2047] * 8)}
    for label, ctx in cases.items():
        rows = int(ctx.lengths.sum())
        x = torch.randn(rows, width, device="cuda", dtype=f32)
        delta = torch.randn(rows, width, device="cuda", dtype=f32)
        vector = lambda: torch.randn(width, device="cuda")      # noqa: E731
        pair, post = (vector(), vector()), (vector(), vector())
        record(f"layer_norm.{label}", _time(lambda: k.layer_norm_step(x, 1e-6, norm=pair, out_dtype=bf16), flush),
               rows * width * 6)
        record(f"add_layer_norm_layer_norm.{label}",
               _time(lambda: k.layer_norm_step(x, 1e-6, delta=delta, delta_norm=post, norm=pair, out_dtype=bf16), flush),
               rows * width * 14)
        xb, db = x.to(bf16), delta.to(bf16)
        record(f"qwen.add_rms_norm.{label}", _time(lambda: k.add_rms_norm(xb, db, None, 1e-6), flush), rows * width * 8)
        # norms, rotation and cache write; queries into the latent space; values out of it
        page, context = 16, int(ctx.positions.max() + ctx.lengths.max())
        pages_per_request = -(-context // page)
        table = torch.arange(ctx.num_segments * pages_per_request, dtype=torch.int32, device="cuda").view(ctx.num_segments, -1)
        pool = torch.randn(ctx.num_segments * pages_per_request, 1, page, rank + rot, device="cuda").to(bf16)
        down = torch.randn(rows, q_rank + rank + rot + heads * vdim, device="cuda")
        positions = torch.cat([torch.arange(int(p), int(p) + int(n), dtype=torch.int32)
                               for p, n in zip(ctx.positions, ctx.lengths)]).cuda()
        slots = torch.cat([torch.arange(int(p), int(p) + int(n), dtype=torch.int64) + i * pages_per_request * page
                           for i, (p, n) in enumerate(zip(ctx.positions, ctx.lengths))]).cuda()
        frequencies = torch.rand(rot // 2, device="cuda")
        wq, wc = torch.ones(q_rank, device="cuda"), torch.ones(rank, device="cuda")
        record(f"latent_prepare.{label}",
               _time(lambda: k.latent_prepare(down, 0, q_rank, q_rank, rank, rot, wq, wc, 1e-6, positions, frequencies,
                                              False, slots, pool), flush),
               rows * ((q_rank + rank + rot) * 4 + (q_rank + rank + rot) * 2))
        qf = torch.randn(rows, heads * (dim + rot), device="cuda")
        w_uk = (torch.randn(heads * dim, rank, device="cuda") * 0.05).to(bf16)
        record(f"absorb_queries.{label}",
               _time(lambda: k.absorb_queries(qf, w_uk, heads, dim, rot, rank, positions, frequencies, False), flush),
               rows * heads * ((dim + rot) * 4 + (rank + rot) * 2) + w_uk.numel() * 2, 2 * rows * heads * dim * rank)
        mixed = torch.randn(rows, heads * rank, device="cuda")
        w_uv = (torch.randn(heads * vdim, rank, device="cuda") * 0.05).to(bf16)
        gate = down[:, q_rank + rank + rot:]
        record(f"latent_values.{label}",
               _time(lambda: k.latent_values(mixed, w_uv, heads, vdim, rank, gate, False), flush),
               rows * heads * (rank * 4 + vdim * 6) + w_uv.numel() * 2, 2 * rows * heads * vdim * rank)
        # attention over a paged cache that already holds every position
        arrays, counts = plan_attention(ctx.lengths, ctx.positions)
        arrays = {name: torch.from_numpy(value).cuda() for name, value in arrays.items()}
        batch = AttentionBatch(ctx.seg_q_start, ctx.seg_q_len, ctx.seg_pos0, ctx.seg_slot, table, ctx.num_segments,
                               ctx.max_q_len, context, arrays, counts)
        qa = (torch.randn(rows, heads * (rank + rot), device="cuda") * 0.2).to(bf16)
        sink = torch.zeros(heads, device="cuda")
        for name, window, sk in (("latent_attention", 0, None), ("latent_attention_windowed", WINDOW, sink)):
            pairs = sum(min(int(p) + i + 1, window) if window else int(p) + i + 1
                        for p, n in zip(ctx.positions, ctx.lengths) for i in range(int(n)))
            keys_read = sum(min(int(p) + int(n), window + int(n)) if window else int(p) + int(n)
                            for p, n in zip(ctx.positions, ctx.lengths))
            record(f"{name}.{label}",
                   _time(lambda: k.latent_attention(qa, pool, batch, heads, rank, rot, 0.08, window, sk), flush),
                   keys_read * (rank + rot) * 2 + rows * heads * ((rank + rot) * 2 + rank * 4),
                   pairs * heads * 2 * (2 * rank + rot))
        # the like kernel of Qwen2: causal attention of the same rows over the same context
        qw = s["qwen"]
        kq = torch.randn(ctx.num_segments * pages_per_request, qw["kv_heads"], page, qw["head_dim"], device="cuda").to(bf16)
        vq = torch.randn_like(kq)
        qq = torch.randn(rows, qw["heads"] * qw["head_dim"], device="cuda").to(bf16)
        full_pairs = sum(int(p) + i + 1 for p, n in zip(ctx.positions, ctx.lengths) for i in range(int(n)))
        record(f"qwen.attention.{label}",
               _time(lambda: k.paged_attention(qq, kq, vq, batch, qw["heads"], qw["kv_heads"], qw["head_dim"],
                                               qw["head_dim"] ** -0.5, None), flush),
               context * ctx.num_segments * qw["kv_heads"] * qw["head_dim"] * 4 + 2 * rows * qw["heads"] * qw["head_dim"] * 2,
               full_pairs * qw["heads"] * 4 * qw["head_dim"])
        # the feed-forward's gate on a product of interleaved blocks, beside the silu gate of the same shape
        gate_up = torch.randn(rows, 2 * s["ff"], device="cuda").to(bf16)
        record(f"clamped_gate.{label}", _time(lambda: k.clamped_gate(gate_up, 64, LIMIT, 1.702), flush), rows * s["ff"] * 6)
        record(f"qwen.swiglu.{label}", _time(lambda: k.swiglu(gate_up, 64), flush), rows * s["ff"] * 6)
        del pool, kq, vq
        torch.cuda.empty_cache()
    k.raise_if_device_error()
    return out


def run(args, host):
    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    peak = host.peaks()
    record = {"metric": "Rozesun beside Qwen2 at equal sizes: prefill of 2,048 tokens and decode at batch 8",
              "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)", "n_gpus": 1,
              "window": WINDOW, "context": 2048, "peaks": peak, "sizes": {}, "kernels": {}}
    with host.ClockSampler() as clocks:
        for size in SIZES:
            entry = {}
            for name, make in (("rozesun", rozesun_config), ("qwen2", qwen_config)):
                config = make(size)
                if name == "rozesun":
                    numbers = rozesun_numbers(config, 2048)
                else:
                    numbers = host.model_numbers(config, config.num_hidden_layers)
                bench = Bench(f"{name} {size}", config, numbers, host)
                entry[name] = model_points(bench, host, args, peak)
                entry[name]["layers"] = len(bench.model.blocks)
                bench.close()
            record["sizes"][size] = entry
            record["kernels"][size] = kernel_points(size, peak)
            print(f"[bench] {size}: {json.dumps(entry)}", file=sys.stderr)
    record["clocks"] = clocks.summary()
    print(json.dumps(record))
    return 0
