"""``bench.py --arch zazasun``: the Zazasun architecture at layer sizes that resemble real models,
beside Qwen2 (the engine's closest model) at equal width, depth and feed-forward size.

Per size: a 2,048-token prefill and decode steps at batch 8 around a context of 2,048 tokens, both
models with random weights in bfloat16, timed on the device (CUDA events, median of the regions;
weights and caches together exceed the L2).  Then each kernel that Zazasun adds, alone, with the
bytes or flops it must move and the fraction of the measured roofline that makes, next to the like
kernel of Qwen2 where there is one.  One JSON line.
"""

from __future__ import annotations

import json
import math
import statistics
import sys
import types

SIZES = {
    # width, feed-forward, groups of (wkv, hgrn2, attention) layers, vocabulary; mixers sized so that
    # every projection has about width rows, as the attention of the Qwen2 model beside it
    "896": dict(width=896, ff=4864, groups=4, vocab=32000,
                attention=dict(heads=7, kv_heads=1, dim=64, vdim=128), wkv=dict(heads=14, dim=64),
                hgrn2=dict(heads=7, dim=128, vdim=128), qwen=dict(heads=14, kv_heads=2, head_dim=64)),
    "2048": dict(width=2048, ff=8192, groups=4, vocab=32000,
                 attention=dict(heads=16, kv_heads=4, dim=64, vdim=128), wkv=dict(heads=32, dim=64),
                 hgrn2=dict(heads=16, dim=128, vdim=128), qwen=dict(heads=16, kv_heads=4, head_dim=128)),
}
WINDOW, KEEP_FIRST = 1024, 4
PREFILL = 2048
MAX_POSITIONS = 8192


def zazasun_config(size):
    from mini_llm_runtime_b200.config import config_from_dict

    s = SIZES[size]
    mlp = {"kind": "dense", "ff": s["ff"]}
    group = [
        {"type": "wkv", "mixer": dict(s["wkv"]), "mlp": mlp},
        {"type": "hgrn2", "mixer": dict(s["hgrn2"]), "mlp": mlp},
        {"type": "attention", "mlp": mlp,
         "mixer": dict(s["attention"], diff=0.5, scale=1.0 / math.sqrt(s["attention"]["dim"]),
                       mask={"size": WINDOW, "keep_first": KEEP_FIRST})},
    ]
    return config_from_dict({"architecture": "Zazasun", "vocab": s["vocab"], "width": s["width"],
                             "max_positions": MAX_POSITIONS, "norm": {"eps": 1e-6}, "layers": group * s["groups"]})


def qwen_config(size):
    from mini_llm_runtime_b200.config import Qwen2Config

    s = SIZES[size]
    return Qwen2Config(vocab_size=s["vocab"], hidden_size=s["width"], intermediate_size=s["ff"],
                       num_hidden_layers=3 * s["groups"], num_attention_heads=s["qwen"]["heads"],
                       num_key_value_heads=s["qwen"]["kv_heads"], head_dim=s["qwen"]["head_dim"],
                       max_position_embeddings=MAX_POSITIONS, rms_norm_eps=1e-6, rope_theta=1e6, hidden_act="silu",
                       tie_word_embeddings=False)


def zazasun_numbers(config, context):
    """Bytes a decode step must read and flops of a prefill, from the configuration."""
    width = config.width
    matrices = 0          # elements of all matrices a token passes through
    cache_bytes = 0       # per request and decode step: keys and values read, states read and written
    mixer_flops = lambda rows: 0     # noqa: E731
    terms = []
    for layer in config.layers:
        a = layer.mixer_args
        if layer.type == "attention":
            rows = 2 * a["heads"] * a["dim"] + 2 * a["kv_heads"] * a["dim"] + a["kv_heads"] * a["vdim"]
            matrices += rows * width + width * a["heads"] * a["vdim"]
            keys = min(context, a["window"] + a["keep_first"]) if a["window"] else context
            cache_bytes += keys * a["kv_heads"] * (2 * a["dim"] + a["vdim"]) * 2
            terms.append(("attention", a))
        elif layer.type == "wkv":
            inner = a["heads"] * a["dim"]
            matrices += 5 * inner * width + max(16, width // 16) * (width + inner)
            cache_bytes += 2 * 4 * inner * a["dim"]
            terms.append(("wkv", a))
        else:
            inner, values = a["heads"] * a["dim"], a["heads"] * a["vdim"]
            matrices += (2 * inner + values) * width + width * values
            cache_bytes += 2 * 4 * inner * a["vdim"]
            terms.append(("hgrn2", a))
        matrices += 3 * width * layer.ff

    def sequence_flops(rows):
        total = 0
        for kind, a in terms:
            if kind == "attention":
                pairs = sum(min(p + 1, a["window"] + a["keep_first"]) for p in range(rows))
                total += pairs * a["heads"] * 4 * (a["dim"] + a["vdim"])
            elif kind == "wkv":
                total += rows * a["heads"] * a["dim"] * a["dim"] * 6
            else:
                total += rows * a["heads"] * a["dim"] * a["vdim"] * 4
        return total

    head = config.vocab * width
    return {"weight_bytes": 2 * (matrices + head), "kv_bytes_per_token": 0, "cache_bytes_per_request": cache_bytes,
            "linear_flops_per_token": 2 * matrices, "head_flops_per_row": 2 * head,
            "attention_flops": lambda rows, before=0: sequence_flops(rows)}


class Bench:
    """What bench.py's timing functions need of a model: config, model, numbers, runner()."""

    def __init__(self, name, config, numbers, host):
        import torch

        from mini_llm_runtime_b200.models import random_model

        self.size = name
        self.config = config
        self.host = host
        self.model = random_model(config, seed=0, dtype=torch.bfloat16, device="cuda:0", draw_on_device=True)
        self.numbers = numbers

    def runner(self, max_requests, tokens_per_request, pages=None):
        import torch

        from mini_llm_runtime_b200.cache import CacheManager
        from mini_llm_runtime_b200.engine import ModelRunner

        block = self.host.BLOCK_SIZE
        pages = pages or max_requests * -(-tokens_per_request // block)
        cache = CacheManager(self.model.cache_needs(), page_size=block, num_pages=pages, max_requests=max_requests,
                             max_tokens_per_request=tokens_per_request, dtype=torch.bfloat16, device="cuda:0",
                             max_step_tokens=PREFILL)
        cache.backup_state = False      # as a server that never retries a failed step would run it
        return ModelRunner(self.model, cache)

    def close(self):
        import torch

        self.model = None
        torch.cuda.empty_cache()


def model_points(bench, host, args, peak, batch=8, context=2048):
    import torch

    prefill_ms, flops, samples = host.time_prefill(bench, repeats=3, warmup=2)
    steps = min(args.steps, 32)
    point = host.decode_point(bench, batch, steps, max(3, args.warmup), 3, context_mean=context, real_prefill=True)
    step_bytes = bench.numbers["weight_bytes"] + batch * (
        context * bench.numbers["kv_bytes_per_token"] + bench.numbers.get("cache_bytes_per_request", 0))
    torch.cuda.empty_cache()
    return {"prefill_2048_ms": round(prefill_ms, 3), "prefill_tokens_per_s": round(PREFILL / prefill_ms * 1e3, 1),
            "prefill_frac_of_bf16_peak": round(flops / (prefill_ms / 1e3) / (peak["bf16_tflops"] * 1e12), 4),
            "decode_b8_ms_per_step": round(point["ms_per_step"], 4),
            "decode_b8_tokens_per_s": round(point["tokens_per_s"], 1),
            "decode_b8_hbm_frac": round(step_bytes / (point["ms_per_step"] / 1e3) / 1e9 / peak["hbm_gbs"], 4),
            "launches_per_region": point["launches"]}


# ---------------------------------------------------------------------------- kernels alone
def _time(call, flush, repeats=5, inner=4):
    """Median device time of one call in microseconds.  The call is captured into a CUDA graph
    ``inner`` times, each time behind a pass that overwrites the L2, and the graph of those passes
    alone is timed and taken off: no host launch time is in the number."""
    import torch

    for _ in range(2):
        call()
    torch.cuda.synchronize()

    def graph_of(with_call):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(inner):
                flush.add_(1)
                if with_call:
                    call()
        return graph

    def median_ms(graph):
        samples = []
        for _ in range(repeats + 1):
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            end.record()
            torch.cuda.synchronize()
            samples.append(start.elapsed_time(end))
        return statistics.median(samples[1:])

    both, alone = graph_of(True), graph_of(False)
    return max(0.0, median_ms(both) - median_ms(alone)) * 1e3 / inner


def _segments(lengths, positions, slots=None):
    import numpy as np
    import torch

    lengths = np.asarray(lengths, dtype=np.int32)
    starts = np.zeros_like(lengths)
    np.cumsum(lengths[:-1], out=starts[1:])
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).cuda()      # noqa: E731
    slots = np.arange(len(lengths)) if slots is None else slots
    return types.SimpleNamespace(seg_q_start=dev(starts), seg_q_len=dev(lengths), seg_pos0=dev(positions),
                                 seg_slot=dev(slots), num_segments=len(lengths), max_q_len=int(lengths.max()),
                                 lengths=lengths, positions=np.asarray(positions, dtype=np.int32))


def kernel_points(size, peak):
    """Each new kernel alone: 2,048 rows of one request (prefill) and 8 requests of one row (decode)."""
    import numpy as np
    import torch

    from mini_llm_runtime_b200 import ops
    from mini_llm_runtime_b200.ops.cuda_ops import AttentionBatch, plan_attention

    k = ops.current()
    s = SIZES[size]
    width = s["width"]
    flush = torch.zeros(96 << 20, dtype=torch.float32, device="cuda")      # 384 MB, three times the L2
    bf16, f32 = torch.bfloat16, torch.float32
    hbm = peak["hbm_gbs"] * 1e9
    out = {}

    def record(name, micros, nbytes=None, flops=None, note=None):
        entry = {"us": round(micros, 2)}
        if nbytes is not None:
            entry["bytes"] = int(nbytes)
            entry["hbm_frac"] = round(nbytes / (micros * 1e-6) / hbm, 4)
        if flops is not None:
            entry["tflops"] = round(flops / (micros * 1e-6) / 1e12, 3)
            entry["bf16_peak_frac"] = round(flops / (micros * 1e-6) / (peak["bf16_tflops"] * 1e12), 5)
        if note:
            entry["note"] = note
        out[name] = entry

    cases = {"prefill": _segments([PREFILL], [0]), "decode": _segments([1] * 8, [2047] * 8)}
    for label, ctx in cases.items():
        rows = int(ctx.lengths.sum())
        x = torch.randn(rows, width, device="cuda", dtype=f32)
        gain = torch.ones(1, device="cuda")
        record(f"scalar_rms_norm.{label}", _time(lambda: k.scalar_rms_norm(x, gain, 1e-6, bf16, want_float=True), flush),
               rows * width * 10)
        xb = x.to(bf16)
        record(f"qwen.rms_norm.{label}", _time(lambda: k.rms_norm(xb, None, 1e-6), flush), rows * width * 4)
        state = torch.zeros(8, width, device="cuda")
        for n in (1, 5):
            coef = torch.rand(n, width, device="cuda")
            record(f"token_shift_x{n}.{label}", _time(lambda: k.token_shift(x, coef, state, ctx, bf16), flush),
                   rows * width * (4 + 2 * n))
        # recurrences
        a = s["wkv"]
        inner = a["heads"] * a["dim"]
        r, key, v, raw, gate = (torch.randn(rows, inner, device="cuda") * 0.3 for _ in range(5))
        bias, bonus, weight = (torch.randn(inner, device="cuda") * 0.1 for _ in range(3))
        st = torch.zeros(8, a["heads"], a["dim"], a["dim"], device="cuda")
        nbytes = rows * inner * (5 * 4 + 2) + 2 * ctx.num_segments * inner * a["dim"] * 4
        record(f"bonus_recurrence.{label}",
               _time(lambda: k.bonus_recurrence(r, key, v, raw, gate, bias, bonus, weight, 1e-6, st, ctx, a["heads"],
                                                a["dim"], bf16), flush),
               nbytes, rows * inner * a["dim"] * 6)
        a = s["hgrn2"]
        inner, values = a["heads"] * a["dim"], a["heads"] * a["vdim"]
        q, f = (torch.randn(rows, inner, device="cuda") * 0.3 for _ in range(2))
        v = torch.randn(rows, values, device="cuda") * 0.3
        bias, lower = torch.randn(inner, device="cuda") * 0.1, torch.rand(inner, device="cuda")
        weight = torch.ones(a["vdim"], device="cuda")
        st = torch.zeros(8, a["heads"], a["dim"], a["vdim"], device="cuda")
        nbytes = rows * (2 * inner * 4 + values * 4 + values * 2) + 2 * ctx.num_segments * inner * a["vdim"] * 4
        record(f"forget_gate_recurrence.{label}",
               _time(lambda: k.forget_gate_recurrence(q, f, v, bias, lower, weight, 1e-6, st, ctx, a["heads"], a["dim"],
                                                      a["vdim"], bf16), flush),
               nbytes, rows * inner * a["vdim"] * 4)
        # differential attention over a paged cache that already holds every position
        a = s["attention"]
        page, context = 16, int(ctx.positions.max() + ctx.lengths.max())
        pages_per_request = -(-context // page)
        table = torch.arange(ctx.num_segments * pages_per_request, dtype=torch.int32, device="cuda").view(ctx.num_segments, -1)
        k_pool = (torch.randn(ctx.num_segments * pages_per_request, a["kv_heads"], page, 2 * a["dim"], device="cuda")).to(bf16)
        v_pool = (torch.randn(ctx.num_segments * pages_per_request, a["kv_heads"], page, a["vdim"], device="cuda")).to(bf16)
        arrays, counts = plan_attention(ctx.lengths, ctx.positions)
        arrays = {name: torch.from_numpy(value).cuda() for name, value in arrays.items()}
        batch = AttentionBatch(ctx.seg_q_start, ctx.seg_q_len, ctx.seg_pos0, ctx.seg_slot, table, ctx.num_segments,
                               ctx.max_q_len, context, arrays, counts)
        qn = torch.randn(rows, 2 * a["heads"] * a["dim"], device="cuda").to(bf16)
        pairs = sum(min(int(p) + i + 1, WINDOW + KEEP_FIRST) for p, n in zip(ctx.positions, ctx.lengths) for i in range(int(n)))
        flops = pairs * a["heads"] * 4 * (a["dim"] + a["vdim"])
        keys_read = sum(min(int(p) + int(n), WINDOW + KEEP_FIRST + int(n)) for p, n in zip(ctx.positions, ctx.lengths))
        nbytes = keys_read * a["kv_heads"] * (2 * a["dim"] + a["vdim"]) * 2 + rows * a["heads"] * (2 * a["dim"] + a["vdim"]) * 2
        record(f"differential_attention.{label}",
               _time(lambda: k.differential_attention(qn, k_pool, v_pool, batch, a["heads"], a["kv_heads"], a["dim"],
                                                      a["vdim"], 0.125, WINDOW, KEEP_FIRST, 0.4, 1e-6, 0.5), flush),
               nbytes, flops)
        qkv = torch.randn(rows, 2 * a["heads"] * a["dim"] + a["kv_heads"] * (2 * a["dim"] + a["vdim"]), device="cuda")
        slots = torch.arange(rows, dtype=torch.int64, device="cuda")
        wq = torch.ones(a["dim"], device="cuda")
        record(f"qk_norm_kv_write.{label}",
               _time(lambda: k.qk_norm_kv_write(qkv, wq, wq, 1e-6, slots, k_pool, v_pool, a["heads"], a["kv_heads"],
                                                a["dim"], a["vdim"]), flush), qkv.numel() * 6)
        # the like kernel of Qwen2: causal attention of the same rows over the same context
        qa = s["qwen"]
        kq = (torch.randn(ctx.num_segments * pages_per_request, qa["kv_heads"], page, qa["head_dim"], device="cuda")).to(bf16)
        vq = torch.randn_like(kq)
        qq = torch.randn(rows, qa["heads"] * qa["head_dim"], device="cuda").to(bf16)
        full_pairs = sum(int(p) + i + 1 for p, n in zip(ctx.positions, ctx.lengths) for i in range(int(n)))
        nbytes = context * ctx.num_segments * qa["kv_heads"] * qa["head_dim"] * 4 + 2 * rows * qa["heads"] * qa["head_dim"] * 2
        record(f"qwen.attention.{label}",
               _time(lambda: k.paged_attention(qq, kq, vq, batch, qa["heads"], qa["kv_heads"], qa["head_dim"],
                                               qa["head_dim"] ** -0.5, None), flush),
               nbytes, full_pairs * qa["heads"] * 4 * qa["head_dim"])
        del k_pool, v_pool, kq, vq
        torch.cuda.empty_cache()
    k.raise_if_device_error()
    return out


def run(args, host):
    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    peak = host.peaks()
    record = {"metric": "Zazasun beside Qwen2 at equal sizes: prefill of 2,048 tokens and decode at batch 8",
              "dtype": "bf16", "data": "synthetic (seeded random weights and token ids)", "n_gpus": 1,
              "window": WINDOW, "keep_first": KEEP_FIRST, "context": 2048, "peaks": peak, "sizes": {}, "kernels": {}}
    with host.ClockSampler() as clocks:
        for size in SIZES:
            entry = {}
            for name, make, numbers in (("zazasun", zazasun_config, None), ("qwen2", qwen_config, None)):
                config = make(size)
                if name == "zazasun":
                    numbers = zazasun_numbers(config, 2048)
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
