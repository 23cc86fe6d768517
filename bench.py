"""Benchmark of the engine on one B200: decode tokens per second at the Qwen3-8B shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference] [--shape 8b|14b|32b|sukalorn|zifuzen|renadra|zavizen]

Prints ONE JSON line.  A "step" is one decode step of the whole batch through the engine's own step
function (every kernel of the model and the token choice); ``value`` is batch / step time, timed with CUDA
events around K steps.  ``e2e`` is the same quantity through the Python entry point's scheduler loop: every
step copies that step's token ids and index data from pinned host memory to the device and reads the
chosen tokens back.  ``prefill`` is one 2,048-token prompt in one step; ``points`` holds decode at batch 1
and 64; ``roofline`` compares the bytes a decode step must read (every weight once, the live requests'
cache) with the copy bandwidth.  Weights are random (seeded), token ids synthetic (seeded uniform).
``--shape zifuzen`` does for the Zifuzen design what ``--shape sukalorn`` does for Sukalorn.
``--shape renadra`` sets four Renadra layers beside Zifuzen layers of equal size with dense feed-forwards, and
Renadra's kernels alone beside the like kernels of the other designs.
``--shape zavizen`` sets four Zavizen layers beside Renadra layers of equal size, and Zavizen's kernels alone beside the
like kernels of the other designs.
``--shape sukalorn`` prints a line of its own: prefill and decode of four Sukalorn layers at two sizes beside Qwen3
layers of equal size, and the attention kernels alone.
Between timed steps nothing is flushed: every step streams the whole model (16 GB at full depth) through
a 126 MB L2, so the inputs are larger than L2.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: Qwen3-8B shape
QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "max_position_embeddings": 40960, "tie_word_embeddings": False,
    "hidden_act": "silu", "attention_bias": False,
}
# BASELINE.json configs[3] and [4]: the further sizes (`--shape 14b|32b`), each with its own workload
QWEN3_14B = dict(QWEN3_8B, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, intermediate_size=17408)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600)
SHAPES = {"8b": QWEN3_8B, "14b": QWEN3_14B, "32b": QWEN3_32B}
LONG_CONTEXT = 32768    # 32b: decode at batch 16 with prompts of this many tokens ...
LONG_BATCH = 16
LONG_CHUNK = 2048       # ... prefilled in portions of this many
SERVING_CONTEXT_14B = 16384
CONTEXT = 8192          # the engine's context limit in this run
PROMPT_LEN = 1024       # decode starts from 1,024-token prompts
GEN_LEN = 256
PREFILL_TOKENS = 2048
PAGE_SIZE = 16
SERVING_REQUESTS = 64               # the scheduler load: this many requests ...
SERVING_PROMPT = (128, 4096)        # ... with prompts of uniformly drawn lengths in this range
SERVING_OUTPUT = (128, 512)         # ... and this many generated tokens each
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as handle:
                raw = json.load(handle)
            flat = {}

            def walk(d):
                for k, v in d.items():
                    if isinstance(v, dict):
                        walk(v)
                    elif isinstance(v, (int, float)) and k not in flat:
                        flat[k] = float(v)
            walk(raw)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                flat["source"] = "measured"
                return flat
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int = 0):
        self.samples: list[list[str]] = []
        self.proc = None
        self.index = index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        mhz = [int(s[0]) for s in self.samples if s[0].isdigit()]
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        reasons = sorted({name for s in self.samples for name, flag in zip(self.NAMES, s[2:]) if flag == "Active"})
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


def model_numbers(cfg: dict, layers: int) -> dict:
    h, nh, nkv, d, i, v = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                           cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"])
    per_layer = (nh + 2 * nkv) * d * h + h * nh * d + 3 * i * h
    return {"layer_params": per_layer, "head_params": v * h, "layer_norm_params": 2 * h + 2 * d,
            "kv_bytes_per_token": 2 * nkv * d * 2 * layers}


def decode_bytes(cfg, layers, batch, mean_ctx) -> float:
    n = model_numbers(cfg, layers)
    weights = 2.0 * (layers * n["layer_params"] + n["head_params"]) + 4.0 * (layers * n["layer_norm_params"])
    return weights + batch * mean_ctx * n["kv_bytes_per_token"]


def prefill_flops(cfg, layers, tokens) -> dict:
    n = model_numbers(cfg, layers)
    gemm = 2.0 * tokens * layers * n["layer_params"] + 2.0 * n["head_params"]
    attn = 4.0 * cfg["num_attention_heads"] * cfg["head_dim"] * layers * tokens * (tokens + 1) / 2
    return {"gemm": gemm, "attention": attn}


def reference_arm(args) -> int:
    """The unmodified reference project (installed under baseline/_ref) on its stock default path.

    Its loader needs the published checkpoint and its extension holds sm_86 code only, but its default generation
    path needs neither: ``ampere_kv.runner.generate_tokens(model, input_ids, cache_kind="contiguous")``
    (ampere_kv/runner.py:301-406; ``--cache contiguous`` is the command line's default, runner.py:667) takes the
    model as an argument and reads weights off it by attribute.  A tree of ``types.SimpleNamespace`` with exactly
    those attributes, holding seeded random bfloat16 tensors of the Qwen3-8B sizes, stands in for the checkpoint.
    The reference without its extension decodes one request at a time, so a "step" of the batch is one token for
    each of the batch's requests in turn.  Nothing of this repository's package is imported here.
    """
    import traceback
    import types
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    cfg = dict(QWEN3_8B)
    cfg["num_hidden_layers"] = args.layers
    steps, warmup, batch = args.steps, max(3, args.warmup), args.batch
    try:
        if not os.path.isdir(os.path.join(ref_root, "ampere_kv")):
            raise RuntimeError("baseline/_ref/ampere_kv is missing (the offline install did not travel)")
        sys.path.insert(0, ref_root)
        sys.dont_write_bytecode = True
        os.environ.setdefault("HF_HUB_OFFLINE", "1")
        import torch
        from ampere_kv import runner as ref           # imports the checkpoint library at module level
        device = torch.device("cuda:0")
        torch.cuda.set_device(device)
        gen = torch.Generator(device=device).manual_seed(0)
        h, nh, nkv, d, inter, vocab = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                                       cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"])
        ns = types.SimpleNamespace

        def matrix(rows, cols):
            return (torch.randn((rows, cols), generator=gen, device=device, dtype=torch.float32) * 0.02).bfloat16()

        def lin(rows, cols):
            return ns(weight=matrix(rows, cols), bias=None)

        def norm(size):
            w = 1.0 + 0.1 * torch.randn((size,), generator=gen, device=device, dtype=torch.float32)
            return ns(weight=w.bfloat16(), variance_epsilon=cfg["rms_norm_eps"])

        layers = []
        for _ in range(args.layers):
            attn = ns(q_proj=lin(nh * d, h), k_proj=lin(nkv * d, h), v_proj=lin(nkv * d, h), o_proj=lin(h, nh * d),
                      q_norm=norm(d), k_norm=norm(d), head_dim=d, sliding_window=None)
            mlp = ns(gate_proj=lin(inter, h), up_proj=lin(inter, h), down_proj=lin(h, inter))
            layers.append(ns(self_attn=attn, mlp=mlp, input_layernorm=norm(h), post_attention_layernorm=norm(h)))
        exponent = torch.arange(0, d, 2, dtype=torch.int64).float() / d
        model = ns(model=ns(embed_tokens=ns(weight=matrix(vocab, h)), layers=layers, norm=norm(h)),
                   lm_head=lin(vocab, h),
                   config=ns(head_dim=d, num_key_value_heads=nkv, rope_theta=cfg["rope_theta"], hidden_act="silu"),
                   _ampere_inv_freq=(1.0 / (cfg["rope_theta"] ** exponent)).to(device),
                   generation_config=ns(eos_token_id=None))
        host_gen = torch.Generator().manual_seed(1234)
        prompts = [torch.randint(0, vocab, (1, PROMPT_LEN), generator=host_gen).pin_memory() for _ in range(batch)]

        def run(prompt_host, new_tokens, timings=None):
            ids = prompt_host.to(device, non_blocking=True)
            return ref.generate_tokens(model, ids, max_new_tokens=new_tokens, cache_kind="contiguous",
                                       ignore_eos=True, timings=timings)

        def device_ms(prompt_host, new_tokens):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            run(prompt_host, new_tokens)
            stop.record()
            torch.cuda.synchronize()
            return start.elapsed_time(stop)

        run(prompts[0], 4)                       # library handles, kernels loaded
        with ClockSampler() as clocks:
            step_ms = e2e_step_ms = 0.0
            for prompt in prompts:
                # the K timed decode steps of this request: a run of 1 + W + K tokens less a run of 1 + W tokens
                short = min(device_ms(prompt, 1 + warmup) for _ in range(2))
                timings: dict = {}
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                start.record()
                run(prompt, 1 + warmup + steps, timings)
                stop.record()
                torch.cuda.synchronize()
                step_ms += (start.elapsed_time(stop) - short) / steps
                e2e_step_ms += timings["tpot_ms"]        # its own host clock: token ids on the host every step
        clock_summary = clocks.summary()
        # prefill: the time to the first token of a 2,048-token prompt, by the reference's own clock
        long_prompt = torch.randint(0, vocab, (1, PREFILL_TOKENS), generator=host_gen).pin_memory()
        run(long_prompt, 1)
        ttft = []
        for _ in range(3):
            timings = {}
            run(long_prompt, 1, timings)
            ttft.append(timings["ttft_ms"])
        prefill_ms = statistics.median(ttft)
        peaks = load_peaks()
        flops = prefill_flops(cfg, args.layers, PREFILL_TOKENS)
        line = {
            "impl": "reference",
            "metric": "decode tok/s at batch 8 (Qwen3-8B shape, B200); prefill alongside",
            "value": round(batch / (step_ms / 1000), 2), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
            "warmup": warmup, "ms_per_step": round(step_ms, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded uniform token ids, seeded random weights)",
            "config": {
                "model": "Qwen3-8B shape", "layers": args.layers, "layers_full": QWEN3_8B["num_hidden_layers"],
                "hidden": h, "heads": nh, "kv_heads": nkv, "head_dim": d, "intermediate": inter, "vocab": vocab,
                "global_batch": batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN,
                "path": "ampere_kv.runner.generate_tokens, cache_kind=contiguous (its default), SDPA, no extension",
                "batching": "one request at a time (its batched decode needs its sm_86 extension)",
                "timing": "CUDA events: run of 1+W+K tokens less run of 1+W tokens, per request, summed",
                "parallelism": "single GPU", "l2": "inputs larger than L2 (all weights stream every token)",
            },
            "e2e": {"value": round(batch / (e2e_step_ms / 1000), 2), "unit": "tokens/s",
                    "ms_per_step": round(e2e_step_ms, 4), "h2d_bytes_per_step": 8 * batch,
                    "d2h_bytes_per_step": 8 * batch},
            "gpu_launches": 0,
            "prefill": {"value": round(PREFILL_TOKENS / (prefill_ms / 1000), 1), "tokens": PREFILL_TOKENS,
                        "ms": round(prefill_ms, 3),
                        "frac": round(flops["gemm"] / (prefill_ms / 1000) / (peaks["bf16_tflops"] * 1e12), 4)},
            "clocks": clock_summary,
        }
        print(json.dumps(line))
        return 0
    except BaseException as exc:        # the actual error goes on record instead of a guess
        if isinstance(exc, KeyboardInterrupt):
            raise
        last = traceback.format_exception_only(type(exc), exc)[-1].strip()
        where = traceback.extract_tb(exc.__traceback__)[-1]
        print(json.dumps({"impl": "reference", "unavailable":
                          f"{last} (at {os.path.basename(where.filename)}:{where.lineno})"[:400]}))
        return 0


def serving_load(engine, synthetic, num_requests, prompt_range, output_range, seed=7) -> dict:
    """A scheduler load: many requests of mixed lengths, chunked prefill beside decoding, host tokens in and out.
    Two passes; the second is timed (the decode graphs of its batch sizes exist by then).  Throughput by the wall
    clock, and per request the time to its first token and its longest wait between two tokens."""
    import random
    import torch
    rng = random.Random(seed)
    lengths = [(rng.randint(*prompt_range), rng.randint(*output_range)) for _ in range(num_requests)]
    for timed_pass in (False, True):
        scheduler = engine.new_scheduler(record_times=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        requests = [scheduler.submit(f"s{i}", synthetic(n_in), n_out, ignore_eos=True)
                    for i, (n_in, n_out) in enumerate(lengths)]
        while scheduler.has_work():
            scheduler.step()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        assert all(len(r.output_ids) == n_out for r, (_, n_out) in zip(requests, lengths))
    ttft = sorted(r.ttft_ms for r in requests)
    gaps = sorted(r.largest_gap_ms for r in requests if r.largest_gap_ms is not None)
    return {"serving_requests": num_requests,
            "serving_output_tok_s": round(sum(n for _, n in lengths) / wall, 1),
            "serving_total_tok_s": round(sum(a + b for a, b in lengths) / wall, 1),
            "serving_rounds": scheduler.rounds,
            "serving_ttft_ms_median": round(ttft[len(ttft) // 2], 1), "serving_ttft_ms_max": round(ttft[-1], 1),
            "serving_largest_gap_ms_median": round(gaps[len(gaps) // 2], 2),
            "serving_largest_gap_ms_max": round(gaps[-1], 2)}


def insert_point(engine, synthetic, batch, prompt_len=PROMPT_LEN, insert_len=PREFILL_TOKENS) -> dict:
    """``batch`` requests decode; a prompt of ``insert_len`` tokens arrives.  Its time to the first token, the
    longest token-to-token wait of the running requests while it is prefilled, and their usual one."""
    import torch
    scheduler = engine.new_scheduler(record_times=True)
    running = [scheduler.submit(f"i{i}", synthetic(prompt_len), 96, ignore_eos=True) for i in range(batch)]
    while any(len(r.output_ids) < 24 for r in running):
        scheduler.step()
    torch.cuda.synchronize()
    newcomer = scheduler.submit("newcomer", synthetic(insert_len), 4, ignore_eos=True)
    while scheduler.has_work():
        scheduler.step()
    gaps = sorted(b - a for r in running for a, b in zip(r.token_times[8:], r.token_times[9:]))
    return {"insert_prompt_tokens": insert_len, "insert_ttft_ms": round(newcomer.ttft_ms, 2),
            "insert_running_gap_ms_max": round(max(r.largest_gap_ms for r in running), 2),
            "insert_running_gap_ms_median": round(gaps[len(gaps) // 2] * 1000, 3)}


def _shape_setup(args, shape_cfg, *, pool_tokens, max_seqs, max_context):
    import torch
    from ampere_kv_engine_b200.config.engine_config import EngineConfig
    from ampere_kv_engine_b200.engine.engine import Engine
    cfg = dict(shape_cfg)
    cfg["num_hidden_layers"] = args.layers
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    engine = Engine.from_random(cfg, seed=0, device=device, config=EngineConfig(
        dtype="bfloat16", page_size=args.page_size, max_tokens=pool_tokens, max_seqs=max_seqs,
        max_batch_tokens=PREFILL_TOKENS, max_context=max_context))
    gen = torch.Generator().manual_seed(1234)
    vocab = cfg["vocab_size"]
    return cfg, engine, (lambda n: torch.randint(0, vocab, (n,), generator=gen).tolist())


def _shape_config(cfg, args, full_layers, **more) -> dict:
    out = {"layers": args.layers, "layers_full": full_layers, "hidden": cfg["hidden_size"],
           "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
           "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "page_size": args.page_size,
           "kv_dtype": "bf16", "parallelism": "single GPU"}
    out.update(more)
    return out


def serving_shape(args) -> int:
    """Qwen3-14B sizes: 64 requests, prompts of 128 to 4,096 tokens, 128 to 512 new tokens each, rounds of at most
    2,048 tokens, 16,384 positions of context.  ``value`` is generated tokens per second of the whole load."""
    pool = SERVING_REQUESTS * (SERVING_PROMPT[1] + SERVING_OUTPUT[1]) // 2 + SERVING_REQUESTS * 64
    cfg, engine, synthetic = _shape_setup(args, QWEN3_14B, pool_tokens=pool, max_seqs=SERVING_REQUESTS + 2,
                                          max_context=SERVING_CONTEXT_14B)
    with ClockSampler() as clocks:
        serving = serving_load(engine, synthetic, SERVING_REQUESTS, SERVING_PROMPT, SERVING_OUTPUT)
    line = {"metric": "generated tok/s of a mixed scheduler load (Qwen3-14B shape, B200)",
            "value": serving["serving_output_tok_s"], "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True,
            "dtype": "bf16", "data": "synthetic (seeded uniform token ids, seeded random weights)",
            "config": _shape_config(cfg, args, QWEN3_14B["num_hidden_layers"], model="Qwen3-14B shape",
                                    requests=SERVING_REQUESTS, prompt_tokens="128-4096", new_tokens="128-512",
                                    max_batch_tokens=PREFILL_TOKENS, seq_len=SERVING_CONTEXT_14B),
            "points": serving, "clocks": clocks.summary()}
    print(json.dumps(line))
    return 0


def long_context_shape(args) -> int:
    """Qwen3-32B sizes: 16 requests with 32,768-token prompts, prefilled in portions of 2,048 tokens, then decoded
    together.  At full depth the 16 caches (8.6 GB each) do not fit beside the weights: admission by page budget
    lets as many in as the pool holds and the rest wait; ``value`` is decode tokens per second of the live batch,
    with the bytes it must read over its time as the roofline fraction."""
    import torch
    from ampere_kv_engine_b200.engine.batch import SeqStep
    from ampere_kv_engine_b200.sampling.sampler import SamplingParams
    cfg = dict(QWEN3_32B)
    cfg["num_hidden_layers"] = args.layers
    peaks = load_peaks()
    numbers = model_numbers(cfg, args.layers)
    weight_bytes = 2.0 * (args.layers * numbers["layer_params"] + 2 * numbers["head_params"])
    free_bytes = torch.cuda.mem_get_info(0)[0]
    # every request decodes beside the later ones' prompt portions, so it needs room for those tokens too
    new_tokens = LONG_BATCH * (LONG_CONTEXT // LONG_CHUNK + 1) + args.warmup + args.steps + 8
    per_request = (LONG_CONTEXT + new_tokens + 64) * numbers["kv_bytes_per_token"]
    room = free_bytes - weight_bytes - 12 * 2 ** 30          # activations of a 2,048-token portion, logits, slack
    live = int(max(1, min(LONG_BATCH, room // per_request)))
    cfg, engine, synthetic = _shape_setup(args, QWEN3_32B, pool_tokens=live * (LONG_CONTEXT + new_tokens + 64),
                                          max_seqs=LONG_BATCH + 2, max_context=LONG_CONTEXT + new_tokens)
    runner = engine.runner
    # through the scheduler: all 16 are submitted, the page budget admits `live` of them, the rest wait
    scheduler = engine.new_scheduler(record_times=True)
    requests = [scheduler.submit(f"L{i}", synthetic(LONG_CONTEXT), new_tokens, ignore_eos=True)
                for i in range(LONG_BATCH)]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    prefill_rounds = 0
    while scheduler.prefilling or not scheduler.running:
        scheduler.step()
        prefill_rounds += 1
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    admitted = sum(1 for r in requests if r.seq is not None)
    waiting = len(scheduler.waiting)
    for _ in range(args.warmup):
        scheduler.step()
    with ClockSampler() as clocks:
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        t0 = time.perf_counter()
        stats = None
        for _ in range(args.steps):
            _, stats = scheduler.step()
        stop.record()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1000 / args.steps
        ms = start.elapsed_time(stop) / args.steps
    batch = stats.decode_tokens
    assert stats.prefill_tokens == 0 and batch == admitted
    mean_ctx = sum(r.seq.length for r in requests if r.seq is not None) / batch - args.steps / 2
    bytes_step = decode_bytes(cfg, args.layers, batch, mean_ctx)
    achieved = bytes_step / (ms / 1000) / 1e9
    for r in requests:
        scheduler.cancel(r)
    scheduler.step()
    line = {"metric": "decode tok/s at batch 16 with 32,768-token prompts (Qwen3-32B shape, B200)",
            "value": round(batch / (ms / 1000), 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic (seeded uniform token ids, seeded random weights)",
            "config": _shape_config(cfg, args, QWEN3_32B["num_hidden_layers"], model="Qwen3-32B shape",
                                    global_batch=LONG_BATCH, live_batch=batch, waiting_for_pages=waiting,
                                    mean_decode_context=round(mean_ctx, 1),
                                    seq_len=LONG_CONTEXT, prefill_chunk=LONG_CHUNK),
            "e2e": {"value": round(batch / (e2e_ms / 1000), 2), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4)},
            "prefill": {"tokens": admitted * LONG_CONTEXT, "seconds": round(prefill_s, 2), "rounds": prefill_rounds,
                        "value": round(live * LONG_CONTEXT / prefill_s, 1)},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / peaks["hbm_gbs"], 4), "peaks": peaks["source"]},
            "clocks": clocks.summary()}
    print(json.dumps(line))
    return 0


# Sukalorn at sizes that resemble a real model's layers, and the Qwen3 layers they are set beside: the same width,
# heads, head size and feed-forward width.  Four layers each (Sukalorn: attention, latent, attention, latent).
SUKALORN_SIZES = {
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, q_rank=768, kv_rank=512, rot_dim=64, block=1024),
    "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=12288, q_rank=1536, kv_rank=512, rot_dim=64, block=1024),
}
SUKALORN_VOCAB = 32000
SUKALORN_LAYERS = 4
#: float32 multiply-adds of the CUDA cores, the pipe a recurrence kept in 32-bit runs on: 148 SMs x 128 lanes x 2 FLOPs
#: at the 1,965 MHz the clocks show under load
FP32_FMA_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12


def sukalorn_config(z: dict, layers: int) -> dict:
    attention = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"],
                 "scale": z["dim"] ** -0.5, "softcap": 30.0, "mask": {"size": z["block"]}, "v_mix": True}
    latent = {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot_dim"], "vdim": z["dim"], "q_rank": z["q_rank"],
              "kv_rank": z["kv_rank"], "scale": (z["dim"] + z["rot_dim"]) ** -0.5,
              "rot": {"base": 10000.0, "dims": z["rot_dim"]}}
    mlp = {"kind": "dense", "ff": z["ff"]}
    return {"architecture": "Sukalorn", "vocab": SUKALORN_VOCAB, "width": z["width"], "norm": {"eps": 1e-6},
            "layers": [{"type": "attention" if i % 2 == 0 else "latent_attention",
                        "mixer": dict(attention if i % 2 == 0 else latent), "mlp": dict(mlp)} for i in range(layers)]}


def qwen3_like(z: dict, layers: int) -> dict:
    return dict(QWEN3_8B, num_hidden_layers=layers, hidden_size=z["width"], num_attention_heads=z["heads"],
                num_key_value_heads=z["kv_heads"], head_dim=z["dim"], intermediate_size=z["ff"],
                vocab_size=SUKALORN_VOCAB)


# Zifuzen at sizes that resemble a real model's layers: four layers (delta + routed experts, attention + dense,
# delta_2 + routed experts, attention on the second layer's pages + routed experts), beside Qwen3 layers of the same
# width, heads, head size and dense feed-forward width.  A token's routed experts and the shared one together are as
# wide as half the dense feed-forward.
ZIFUZEN_SIZES = {
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, delta_heads=16, delta_qk_heads=4, conv=4,
               experts=32, top=4, expert_ff=768, shared_ff=1024, groups=(8, 4)),
    "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=12288, delta_heads=32, delta_qk_heads=8, conv=4,
               experts=64, top=4, expert_ff=1024, shared_ff=2048, groups=(8, 4)),
}


def zifuzen_config(z: dict, layers: int) -> dict:
    attention = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"],
                 "scale": z["dim"] ** -0.5}
    delta = {"heads": z["delta_heads"], "kv_heads": z["delta_qk_heads"], "dim": z["dim"], "vdim": z["dim"],
             "conv": z["conv"]}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"], "limit": 7.0},
           "router": {"experts": z["experts"], "top": z["top"], "scale": 2.5,
                      "groups": {"count": z["groups"][0], "keep": z["groups"][1]}},
           "shared": {"ff": z["shared_ff"], "limit": 7.0}}
    dense = {"kind": "dense", "ff": z["ff"]}
    pattern = [("delta", delta, moe), ("attention", attention, dense), ("delta_2", delta, moe),
               ("attention", dict(attention, kv_from=1), moe)]
    out = []
    for i in range(layers):
        kind, mixer, mlp = pattern[i % 4]
        mixer = dict(mixer)
        if "kv_from" in mixer:
            mixer["kv_from"] = i - 2
        out.append({"type": kind, "mixer": mixer, "mlp": json.loads(json.dumps(mlp))})
    return {"architecture": "Zifuzen", "vocab": SUKALORN_VOCAB, "width": z["width"], "max_positions": CONTEXT,
            "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6}, "logit_softcap": 30.0, "layers": out}


# Renadra at sizes that resemble a real model's layers: four layers (hgrn2, attention behind a window, a rotary
# attention with kept first keys and sigmoid weights beside a lightning attention, hgrn2), all with dense feed-forwards,
# beside Zifuzen layers of the same width, heads, head size and feed-forward width (delta rule, attention, delta rule,
# attention; dense feed-forwards): the package's other design with a float32 memory per request and head.
RENADRA_SIZES = {
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, memory_heads=16, window=1024, keep=64),
    "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=12288, memory_heads=32, window=1024, keep=64),
}


def renadra_config(z: dict, layers: int) -> dict:
    d = z["dim"]
    rot = {"base": 1000000.0, "dims": d}
    memory = {"heads": z["memory_heads"], "dim": d, "vdim": d}
    attention = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": d, "vdim": d, "scale": d ** -0.5,
                 "mask": {"size": z["window"]}, "rot": dict(rot)}
    left = dict(attention, softcap=30.0, mask={"size": z["window"], "keep_first": z["keep"]},
                rot=dict(rot, scaling={"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}))
    right = dict(memory, decay=[1.0 - 2.0 ** -(2 + 8 * h / max(1, z["memory_heads"] - 1)) for h in range(z["memory_heads"])])
    parallel = {"left": left, "right": right, "left_scale": 0.8, "right_scale": 1.1}
    mlp = {"kind": "dense", "ff": z["ff"]}
    pattern = [("hgrn2", memory), ("attention", attention), ("parallel", parallel), ("hgrn2", memory)]
    return {"architecture": "Renadra", "vocab": SUKALORN_VOCAB, "width": z["width"], "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0, "bigram": {"buckets": 100003, "mul_prev": 1000003, "mul_cur": 31}},
            "layers": [{"type": pattern[i % 4][0], "mixer": json.loads(json.dumps(pattern[i % 4][1])), "mlp": dict(mlp)}
                       for i in range(layers)]}


# Zavizen at the same sizes: four layers (parallel, mamba2, parallel, mamba2) on four copies of the stream, all with
# dense feed-forwards, beside Renadra's four layers of the same width, heads, head size and feed-forward width: the
# package's other design with mixers side by side, a decaying memory per head and a looped schedule.
ZAVIZEN_STREAMS = 4


def zavizen_config(z: dict, layers: int) -> dict:
    d, h = z["dim"], z["memory_heads"]
    left = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": d, "vdim": d, "scale": d ** -0.5,
            "rot": {"base": 1000000.0, "dims": d // 2, "scaling": {"factor": 4.0}}}
    right = {"heads": h, "dim": d, "vdim": d, "rot": {"base": 1000000.0, "dims": d},
             "decay": [1.0 - 2.0 ** -(2 + 8 * i / max(1, h - 1)) for i in range(h)]}
    mamba = {"heads": h, "vdim": d, "state": d, "groups": 1, "conv": 4, "norm_groups": 1}
    pattern = [("parallel", {"left": left, "right": right}), ("mamba2", mamba)]
    return {"architecture": "Zavizen", "vocab": SUKALORN_VOCAB, "width": z["width"], "norm": {"eps": 1e-6},
            "streams": ZAVIZEN_STREAMS,
            "layers": [{"type": pattern[i % 2][0], "mixer": json.loads(json.dumps(pattern[i % 2][1])),
                        "mlp": {"kind": "dense", "ff": z["ff"]}} for i in range(layers)]}


def zifuzen_dense_like(z: dict, layers: int) -> dict:
    attention = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"],
                 "scale": z["dim"] ** -0.5}
    delta = {"heads": z["memory_heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "conv": 4}
    pattern = [("delta", delta), ("attention", attention), ("delta_2", delta), ("attention", attention)]
    return {"architecture": "Zifuzen", "vocab": SUKALORN_VOCAB, "width": z["width"], "max_positions": CONTEXT,
            "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6}, "logit_softcap": 30.0,
            "layers": [{"type": pattern[i % 4][0], "mixer": dict(pattern[i % 4][1]),
                        "mlp": {"kind": "dense", "ff": z["ff"]}} for i in range(layers)]}


def sukalorn_shape(args, design: str = "sukalorn") -> int:
    """Prefill (one 2,048-token prompt) and decode (batch 8 from 1,024-token prompts) of the Sukalorn design at two
    layer sizes, each beside Qwen3 layers of the same width, heads, head size and feed-forward width, through the
    engine's own step function; then the attention kernels alone at the same shapes, each with the fraction of the
    measured peak it reaches (prompt: FLOPs over the burst bf16 product peak; decode: cache bytes over the copy
    bandwidth).  ``value`` is Sukalorn's decode tokens per second at the larger size.  ``design="zifuzen"``: the same
    for the Zifuzen design, with its delta-rule and routed-expert kernels alone."""
    import torch
    from ampere_kv_engine_b200.config.engine_config import EngineConfig
    from ampere_kv_engine_b200.engine.batch import SeqStep
    from ampere_kv_engine_b200.engine.engine import Engine
    from ampere_kv_engine_b200.kernels import ops
    from ampere_kv_engine_b200.sampling.sampler import SamplingParams
    peaks = load_peaks()
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    layers = args.layers or SUKALORN_LAYERS
    batch = args.batch
    gen = torch.Generator().manual_seed(1234)
    flush = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device=device)      # larger than the 126 MB L2

    def timed(fn, steps, flush_l2=False):
        if not flush_l2:       # whole steps: one pair of events around all of them, the host queues ahead
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for _ in range(steps):
                fn()
            stop.record()
            torch.cuda.synchronize()
            return start.elapsed_time(stop) / steps
        total = 0.0
        for _ in range(steps):
            if flush_l2:
                flush.zero_()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            fn()
            stop.record()
            torch.cuda.synchronize()
            total += start.elapsed_time(stop)
        return total / steps

    def measure(config: dict) -> dict:
        engine = Engine.from_random(config, seed=0, device=device, config=EngineConfig(
            dtype="bfloat16", page_size=args.page_size, max_tokens=(batch + 1) * (PROMPT_LEN + GEN_LEN + 64) + PREFILL_TOKENS,
            max_seqs=batch + 2, max_batch_tokens=PREFILL_TOKENS, max_context=CONTEXT))
        runner, vocab = engine.runner, engine.vocab_size
        synthetic = lambda n: torch.randint(0, vocab, (n,), generator=gen).tolist()
        prompt = synthetic(PREFILL_TOKENS)

        def prefill_once():
            seq = runner.open("prefill")
            logits = runner.step([SeqStep(seq, prompt, [PREFILL_TOKENS - 1])])
            engine.sampler.sample(logits, [SamplingParams()], [0])
            runner.close(seq)

        for _ in range(3):
            prefill_once()
        prefill_ms = timed(prefill_once, 5)
        seqs = [runner.open(f"d{i}") for i in range(batch)]
        for i in range(0, batch, 2):
            runner.step([SeqStep(s, synthetic(PROMPT_LEN), []) for s in seqs[i:i + 2]])
        greedy, zeros = [SamplingParams()] * batch, [0] * batch

        def one():
            logits = runner.step([SeqStep(s, [t], [0]) for s, t in zip(seqs, synthetic(batch))])
            engine.sampler.sample(logits, greedy, zeros)

        for _ in range(args.warmup):
            one()
        ops.launch_count = 0
        decode_ms = timed(one, args.steps)
        launches = ops.launch_count // args.steps
        runner.raise_on_status()
        def matrix_bytes(parts):
            """Bytes of the parts' matrices, a matrix that several parts hold views of counted once."""
            seen, total = set(), 0
            for part in parts:
                for t in vars(part).values():
                    if isinstance(t, torch.Tensor) and t.dim() >= 2:
                        storage = t.untyped_storage()
                        if storage.data_ptr() not in seen:
                            seen.add(storage.data_ptr())
                            total += storage.nbytes()
            return total

        weights = matrix_bytes(engine.model._parts())
        # without the tables a step only gathers rows of (token and pair embeddings): what a decode step reads whole
        from ampere_kv_engine_b200.parts.embedding import Embedding
        read = matrix_bytes(part for part in engine.model._parts() if not isinstance(part, Embedding))
        del engine, runner, seqs
        torch.cuda.empty_cache()
        return {"prefill_ms": round(prefill_ms, 3), "prefill_tok_s": round(PREFILL_TOKENS / prefill_ms * 1000, 1),
                "decode_ms": round(decode_ms, 4), "decode_tok_s": round(batch / decode_ms * 1000, 1),
                "launches_per_decode_step": launches, "matrix_bytes": weights,
                "decode_hbm_frac_weights_only": round(weights / (decode_ms / 1000) / 1e9 / peaks["hbm_gbs"], 4),
                "matrix_bytes_read": read,
                "decode_hbm_frac_matrices_read": round(read / (decode_ms / 1000) / 1e9 / peaks["hbm_gbs"], 4),
                "prefill_matrix_tflops": round(2.0 * (read / 2) * PREFILL_TOKENS / (prefill_ms / 1000) / 1e12, 1)}

    def layout(seq_q, q_tile):
        """Batch layout tensors of sequences given as (context, new tokens): (keyword arguments of the attention ops,
        pages used, tokens)."""
        page = args.page_size
        cu, tiles = [0], []
        for s, (_, n) in enumerate(seq_q):
            tiles += [(s, cu[-1] + t0, min(q_tile, n - t0)) for t0 in range(0, n, q_tile)]
            cu.append(cu[-1] + n)
        pages_per = [(c + page - 1) // page for c, _ in seq_q]
        table = torch.full((len(seq_q), max(pages_per)), -1, dtype=torch.int32)
        at = 0
        for s, n in enumerate(pages_per):
            table[s, :n] = torch.arange(at, at + n, dtype=torch.int32)
            at += n
        dev = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
        return dict(block_table=table.to(device), cu_q=dev(cu), ctx_lens=dev([c for c, _ in seq_q]),
                    tile_seq=dev([t[0] for t in tiles]), tile_q0=dev([t[1] for t in tiles]),
                    tile_nq=dev([t[2] for t in tiles]), num_tiles=len(tiles), q_tile=q_tile), at, cu[-1]

    def kernels_alone(z: dict) -> dict:
        """The attention kernels by themselves at this size: a 2,048-token prompt as one sequence, and single tokens
        of `batch` sequences that each hold 1,024 keys."""
        out = {}
        page, heads, kvh, dim = args.page_size, z["heads"], z["kv_heads"], z["dim"]
        row = z["kv_rank"] + z["rot_dim"]
        bf = dict(dtype=torch.bfloat16, device=device)
        g = torch.Generator(device=device).manual_seed(1)

        for name, seq_q, q_tile in (("prompt", [(PREFILL_TOKENS, PREFILL_TOKENS)], ops.ATTENTION_Q_TILE),
                                    ("decode", [(PROMPT_LEN, 1)] * batch, 1)):
            lay, pages, tokens = layout(seq_q, q_tile)
            keys = sum(c for c, _ in seq_q)
            pairs = sum(n * (2 * c - n + 1) // 2 for c, n in seq_q)           # (query, visible key) pairs, causal
            rand = lambda *shape: torch.randn(shape, generator=g, **bf)
            k_pages, v_pages, rows = rand(pages, kvh, page, dim), rand(pages, kvh, page, dim), rand(pages, 1, page, row)
            q, q_row = rand(tokens, heads * dim), rand(tokens, heads * row)
            slopes = torch.exp2(-8.0 * torch.arange(1, heads + 1, device=device) / heads).float()
            gate = torch.rand((tokens, heads), device=device, generator=g)
            group = heads // kvh
            cases = {
                "qwen3_attention": (lambda s: ops.paged_attention(
                    q, k_pages, v_pages, num_splits=s, num_heads=heads, num_kv_heads=kvh, window=0, scale=dim ** -0.5,
                    **lay), 4.0 * heads * dim * pairs, 2.0 * 2 * kvh * dim * keys,
                    ops.choose_splits(lay["num_tiles"], kvh, q_tile * group, PROMPT_LEN, True) if q_tile == 1 else 1),
                "sukalorn_attention": (lambda s: ops.scored_attention(
                    q, k_pages, v_pages, num_splits=s, num_heads=heads, num_kv_heads=kvh, v_dim=dim, scale=dim ** -0.5,
                    softcap=30.0, slopes=slopes, gate=gate, chunk=0, **lay), 4.0 * heads * dim * pairs,
                    2.0 * 2 * kvh * dim * keys, ops.choose_splits(lay["num_tiles"], kvh, q_tile * group, PROMPT_LEN, False)),
                "sukalorn_latent_attention": (lambda s: ops.scored_attention(
                    q_row, rows, rows, num_splits=s, num_heads=heads, num_kv_heads=1, v_dim=z["kv_rank"],
                    scale=0.07, **lay), 2.0 * heads * (row + z["kv_rank"]) * pairs, 2.0 * row * keys,
                    ops.choose_splits(lay["num_tiles"], 1, q_tile * heads, PROMPT_LEN, False)),
            }
            for case, (fn, flops, cache_bytes, splits) in cases.items():
                for _ in range(3):
                    fn(splits)
                ms = timed(lambda: fn(splits), 5, flush_l2=True)
                entry = {"ms": round(ms, 4), "splits": splits}
                if name == "prompt":
                    entry["tflops"] = round(flops / (ms / 1000) / 1e12, 2)
                    entry["frac_of_bf16_peak"] = round(flops / (ms / 1000) / 1e12 / peaks["bf16_tflops"], 4)
                else:
                    entry["cache_gbs"] = round(cache_bytes / (ms / 1000) / 1e9, 1)
                    entry["frac_of_hbm"] = round(cache_bytes / (ms / 1000) / 1e9 / peaks["hbm_gbs"], 4)
                out[f"{name}_{case}"] = entry
        return out

    def zifuzen_kernels_alone(z: dict) -> dict:
        """The delta rule's scan and the routed experts' grouped products by themselves at this size: a 2,048-token
        prompt as one sequence, and single tokens of `batch` sequences."""
        out = {}
        H, G, D, taps = z["delta_heads"], z["delta_qk_heads"], z["dim"], z["conv"]
        V = D
        channels = 2 * G * D + H * V
        memory, state_floats = ops.delta_state_floats(H, G, D, V, taps)
        g = torch.Generator(device=device).manual_seed(2)
        state = torch.zeros((batch + 1, state_floats), device=device)
        conv = torch.rand((channels, taps), device=device, generator=g) - 0.3
        rate_log = torch.full((H,), -3.0, device=device)
        zeros_h, ones_v = torch.zeros((H,), device=device), torch.ones((V,), device=device)
        sizes_kw = dict(num_heads=H, num_kv_heads=G, head_dim=D, v_dim=V, taps=taps)
        dev = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
        fp32_peak = peaks.get("fp32_tflops") or FP32_FMA_TFLOPS
        for name, lens in (("prompt", [PREFILL_TOKENS]), ("decode", [1] * batch)):
            tokens = sum(lens)
            cu, slots = dev([0] + [sum(lens[:i + 1]) for i in range(len(lens))]), dev(list(range(len(lens))))
            x = torch.randn((tokens, channels + H * V + 2 * H), device=device, generator=g).to(torch.bfloat16)
            prep = lambda: ops.delta_prep(x, conv, rate_log, zeros_h, state, cu, slots, unit_eps=1e-6, **sizes_kw)
            qkv, coef = prep()
            scan = lambda: ops.delta_scan(qkv, coef, x, ones_v, state, cu, slots, norm_eps=1e-6, **sizes_kw)
            for case, fn in (("delta_prep", prep), ("delta_scan", scan)):
                for _ in range(3):
                    fn()
                ms = timed(fn, 5, flush_l2=True)
                entry = {"ms": round(ms, 4)}
                if case == "delta_scan":
                    flops = 7.0 * tokens * H * D * V          # decay, two products and the rank-one update per token
                    moved = 2.0 * 4 * len(lens) * memory + 4.0 * tokens * (channels + 2 * H * V)
                    entry.update(tflops=round(flops / (ms / 1000) / 1e12, 3),
                                 frac_of_fp32_fma_peak=round(flops / (ms / 1000) / 1e12 / fp32_peak, 4),
                                 state_gbs=round(moved / (ms / 1000) / 1e9, 1),
                                 frac_of_hbm=round(moved / (ms / 1000) / 1e9 / peaks["hbm_gbs"], 4))
                out[f"{name}_{case}"] = entry
            # the routed experts: router, choice, sort, both grouped products, the sum
            E, top, F, W = z["experts"], z["top"], z["expert_ff"], z["width"]
            xs = torch.randn((tokens, W), device=device, generator=g).to(torch.bfloat16)
            w_gu = (torch.randn((E, 2 * F, W), device=device, generator=g) * 0.02).to(torch.bfloat16)
            w_d = (torch.randn((E, W, F), device=device, generator=g) * 0.02).to(torch.bfloat16)
            logits = torch.randn((tokens, E), device=device, generator=g)
            route = lambda: ops.moe_route(logits, None, top=top, groups=z["groups"][0], keep_groups=z["groups"][1],
                                          group_top=2, scale=2.5, weight_eps=1e-20)
            chosen, weights = route()
            sort = lambda: ops.moe_sort(chosen, E)
            order, offsets = sort()
            gate_up = lambda: ops.moe_gate_up(xs, w_gu, order, offsets, top=top, limit=7.0, slope=1.702)
            act = gate_up()
            down = lambda: ops.moe_down(act, w_d, order, offsets, weights)
            parts = down()
            used = int((offsets[1:] > offsets[:-1]).sum())
            for case, fn, flops, moved in (
                    ("moe_route", route, 0.0, 4.0 * tokens * E), ("moe_sort", sort, 0.0, 8.0 * tokens * top),
                    ("moe_gate_up", gate_up, 4.0 * tokens * top * F * W, 2.0 * used * 2 * F * W),
                    ("moe_down", down, 2.0 * tokens * top * F * W, 2.0 * used * F * W),
                    ("moe_combine", lambda: ops.moe_combine(parts, None, top=top), 0.0, 4.0 * tokens * (top + 1) * W)):
                for _ in range(3):
                    fn()
                ms = timed(fn, 5, flush_l2=True)
                entry = {"ms": round(ms, 4)}
                if flops:
                    entry.update(tflops=round(flops / (ms / 1000) / 1e12, 2),
                                 frac_of_bf16_peak=round(flops / (ms / 1000) / 1e12 / peaks["bf16_tflops"], 4),
                                 weight_gbs=round(moved / (ms / 1000) / 1e9, 1),
                                 frac_of_hbm=round(moved / (ms / 1000) / 1e9 / peaks["hbm_gbs"], 4))
                out[f"{name}_{case}"] = entry
            # the library product of the same FLOPs as one dense matrix, for scale
            dense_w = w_gu.view(-1, W)[:2 * F * top] if name == "prompt" else None
            if dense_w is not None:
                fn = lambda: torch.nn.functional.linear(xs, dense_w)
                for _ in range(3):
                    fn()
                ms = timed(fn, 5, flush_l2=True)
                flops = 2.0 * tokens * dense_w.shape[0] * W
                out["prompt_library_product_of_equal_flops"] = {
                    "ms": round(ms, 4), "tflops": round(flops / (ms / 1000) / 1e12, 2),
                    "frac_of_bf16_peak": round(flops / (ms / 1000) / 1e12 / peaks["bf16_tflops"], 4)}
        return out

    def renadra_kernels_alone(z: dict) -> dict:
        """Renadra's own kernels by themselves at this size, each beside the like kernel of another design: the
        linear-memory scan in both modes beside the delta rule's scan (all walk a float32 memory per head token by
        token), the norm behind it, the rotary preparation, and the attention with kept first keys and sigmoid weights
        beside the capped, sloped and gated softmax attention of the Sukalorn design and the plain attention behind a
        window.  A 2,048-token prompt as one sequence, and single tokens of `batch` sequences that hold 1,024 keys."""
        out = {}
        H, D, V = z["memory_heads"], z["dim"], z["dim"]
        heads, kvh, dim, page = z["heads"], z["kv_heads"], z["dim"], args.page_size
        window, keep = z["window"], z["keep"]
        g = torch.Generator(device=device).manual_seed(3)
        dev = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
        fp32_peak = peaks.get("fp32_tflops") or FP32_FMA_TFLOPS
        bf = dict(dtype=torch.bfloat16, device=device)
        floats = ops.linear_scan_state_floats(H, D, V)
        taps = 4
        delta_memory, delta_floats = ops.delta_state_floats(H, kvh, D, V, taps)
        state = torch.zeros((batch + 1, max(floats, delta_floats)), device=device)
        lower = torch.rand((H * D,), device=device, generator=g) * 0.9
        gate_bias = torch.zeros((H * D,), device=device)
        decay = torch.tensor(renadra_config(z, 4)["layers"][2]["mixer"]["right"]["decay"], device=device)
        norm_head, norm_wide = torch.ones((V,), device=device), torch.ones((H * V,), device=device)

        def record(key, fn, *, flops=0.0, moved=0.0, tensor=False):
            for _ in range(3):
                fn()
            ms = timed(fn, 5, flush_l2=True)
            entry = {"ms": round(ms, 4)}
            if flops:
                peak = peaks["bf16_tflops"] if tensor else fp32_peak
                entry["tflops"] = round(flops / (ms / 1000) / 1e12, 3)
                entry["frac_of_bf16_peak" if tensor else "frac_of_fp32_fma_peak"] = round(
                    flops / (ms / 1000) / 1e12 / peak, 4)
            if moved:
                entry["gbs"] = round(moved / (ms / 1000) / 1e9, 1)
                entry["frac_of_hbm"] = round(moved / (ms / 1000) / 1e9 / peaks["hbm_gbs"], 4)
            out[key] = entry

        for name, lens in (("prompt", [PREFILL_TOKENS]), ("decode", [1] * batch)):
            tokens = sum(lens)
            cu, slots = dev([0] + [sum(lens[:i + 1]) for i in range(len(lens))]), dev(list(range(len(lens))))
            # the memories: [q | f or k | v | g] columns of one product
            x = torch.randn((tokens, 2 * H * D + 2 * H * V), device=device, generator=g).to(torch.bfloat16)
            sizes_kw = dict(num_heads=H, head_dim=D, v_dim=V, q_off=0, k_off=H * D, v_off=2 * H * D)
            scan_flops = 5.0 * tokens * H * D * V               # decay, write and read of every memory element
            scan_moved = 2.0 * 4 * len(lens) * floats + 2.0 * tokens * 3 * H * D + 4.0 * tokens * H * V
            record(f"{name}_hgrn2_scan", lambda: ops.linear_scan(x, state, cu, slots, mode="gated_write",
                                                                 gate_bias=gate_bias, lower=lower, **sizes_kw),
                   flops=scan_flops, moved=scan_moved)
            record(f"{name}_lightning_scan", lambda: ops.linear_scan(x, state, cu, slots, mode="constant_decay",
                                                                     decay=decay, **sizes_kw),
                   flops=scan_flops, moved=scan_moved)
            o = ops.linear_scan(x, state, cu, slots, mode="constant_decay", decay=decay, **sizes_kw)
            record(f"{name}_norm_per_head", lambda: ops.group_norm_gate(o, norm_head, group=V, eps=1e-6,
                                                                        out_dtype=torch.bfloat16),
                   moved=6.0 * tokens * H * V)
            record(f"{name}_norm_all_heads_gated", lambda: ops.group_norm_gate(
                o, norm_wide, group=H * V, eps=1e-6, out_dtype=torch.bfloat16, x=x, gate_off=2 * H * D + H * V),
                moved=8.0 * tokens * H * V)
            # the like kernel: the delta rule's scan at the same heads and widths
            channels = 2 * kvh * D + H * V
            xd = torch.randn((tokens, channels + H * V + 2 * H), device=device, generator=g).to(torch.bfloat16)
            conv = torch.rand((channels, taps), device=device, generator=g) - 0.3
            delta_kw = dict(num_heads=H, num_kv_heads=kvh, head_dim=D, v_dim=V, taps=taps)
            state.zero_()
            qkv, coef = ops.delta_prep(xd, conv, torch.full((H,), -3.0, device=device), torch.zeros((H,), device=device),
                                       state, cu, slots, unit_eps=1e-6, **delta_kw)
            record(f"{name}_like_delta_scan", lambda: ops.delta_scan(qkv, coef, xd, norm_head, state, cu, slots,
                                                                     norm_eps=1e-6, **delta_kw),
                   flops=7.0 * tokens * H * D * V,
                   moved=2.0 * 4 * len(lens) * delta_memory + 4.0 * tokens * (channels + 2 * H * V))
            state.zero_()
        for name, seq_q, q_tile in (("prompt", [(PREFILL_TOKENS, PREFILL_TOKENS)], ops.ATTENTION_Q_TILE),
                                    ("decode", [(PROMPT_LEN, 1)] * batch, 1)):
            lay, pages, tokens = layout(seq_q, q_tile)
            rand = lambda *shape: torch.randn(shape, generator=g, **bf)
            k_pages, v_pages = rand(pages, kvh, page, dim), rand(pages, kvh, page, dim)
            q = rand(tokens, heads * dim)
            # rotary preparation: reads the product, writes q and both cache rows
            xp = rand(tokens, (heads + kvh) * dim)
            positions = dev([c - n + i for c, n in seq_q for i in range(n)])
            slot_map = dev(list(range(tokens)))
            freq = (1000000.0 ** (-torch.arange(0, dim, 2, device=device).float() / dim)).contiguous()
            record(f"{name}_rotary_prep", lambda: ops.rotary_prep(
                xp, positions, slot_map, freq, k_pages, v_pages, num_heads=heads, num_kv_heads=kvh, head_dim=dim, v_dim=dim,
                rotary_dims=dim, layout="half", factor=1.1, value_from_key=True),
                moved=2.0 * tokens * ((heads + kvh) * dim + heads * dim + 2 * kvh * dim))
            # (query, visible key) pairs behind the window with the kept first keys; keys a decode step reads
            seen = lambda p: min(p + 1, window) + min(keep, max(0, p + 1 - window))
            pairs = sum(seen(c - n + i) for c, n in seq_q for i in range(n))
            keys = sum(seen(c - 1) for c, _ in seq_q)
            pairs_plain = sum(min(c - n + i + 1, window) for c, n in seq_q for i in range(n))
            keys_plain = sum(min(c, window) for c, _ in seq_q)
            group = heads // kvh
            head_bias = torch.zeros((heads,), device=device)
            slopes = torch.exp2(-8.0 * torch.arange(1, heads + 1, device=device) / heads).float()
            gate = torch.rand((tokens, heads), device=device, generator=g)
            reach = window + keep
            tc = ops.scored_takes_tensor_cores(torch.bfloat16, dim, dim, group, page, prompt=q_tile > 1)
            cases = {
                "sigmoid_kept_attention": (lambda s: ops.scored_attention(
                    q, k_pages, v_pages, num_splits=s, num_heads=heads, num_kv_heads=kvh, v_dim=dim, scale=dim ** -0.5,
                    softcap=30.0, window=window, keep_first=keep, sigmoid_weights=True, head_bias=head_bias,
                    out_scale=0.8, **lay), pairs, keys,
                    1 if q_tile > 1 and tc else ops.choose_splits(lay["num_tiles"], kvh, q_tile * group,
                                                                  min(PROMPT_LEN, reach), tc)),
                "window_attention": (lambda s: ops.paged_attention(
                    q, k_pages, v_pages, num_splits=s, num_heads=heads, num_kv_heads=kvh, window=window,
                    scale=dim ** -0.5, **lay), pairs_plain, keys_plain,
                    ops.choose_splits(lay["num_tiles"], kvh, q_tile * group, min(PROMPT_LEN, window), True)
                    if q_tile == 1 else 1),
                "like_sukalorn_attention": (lambda s: ops.scored_attention(
                    q, k_pages, v_pages, num_splits=s, num_heads=heads, num_kv_heads=kvh, v_dim=dim, scale=dim ** -0.5,
                    softcap=30.0, slopes=slopes, gate=gate, window=window, **lay), pairs_plain, keys_plain,
                    1 if q_tile > 1 and tc else ops.choose_splits(lay["num_tiles"], kvh, q_tile * group,
                                                                  min(PROMPT_LEN, window), tc)),
            }
            for case, (fn, n_pairs, n_keys, splits) in cases.items():
                if name == "prompt":
                    record(f"{name}_{case}", lambda: fn(splits), flops=4.0 * heads * dim * n_pairs, tensor=True)
                else:
                    record(f"{name}_{case}", lambda: fn(splits), moved=2.0 * 2 * kvh * dim * n_keys)
                out[f"{name}_{case}"]["splits"] = splits
        return out

    def zavizen_kernels_alone(z: dict) -> dict:
        """The kernels that came with the Zavizen design by themselves at this size, each beside the like kernel of
        another design: the scan on prepared rows with a constant decay and with a decay per token beside the
        lightning scan (Renadra), the state-space preparation beside the delta rule's, the stream's write + read + norm
        beside the residual add + RMS norm, the rotation with norms over whole rows beside the plain rotation, the
        float32 rows, the norm with a skip term and a gate before it beside the gated norm over all heads, two normed
        outputs summed beside the scaled sum.  A 2,048-token prompt as one sequence, and single tokens of `batch`
        sequences."""
        out = {}
        H, D, V, W = z["memory_heads"], z["dim"], z["dim"], z["width"]
        heads, kvh, page = z["heads"], z["kv_heads"], args.page_size
        g = torch.Generator(device=device).manual_seed(3)
        dev = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
        fp32_peak = peaks.get("fp32_tflops") or FP32_FMA_TFLOPS
        floats = ops.linear_scan_state_floats(H, D, V)
        taps, S = 4, ZAVIZEN_STREAMS
        channels = H * V + 2 * D
        delta_memory, delta_floats = ops.delta_state_floats(H, kvh, D, V, taps)
        state = torch.zeros((batch + 1, max(floats + (taps - 1) * channels + 4, delta_floats)), device=device)
        decay = torch.tensor(zavizen_config(z, 2)["layers"][0]["mixer"]["right"]["decay"], device=device)

        def record(key, fn, *, flops=0.0, moved=0.0):
            for _ in range(3):
                fn()
            ms = timed(fn, 5, flush_l2=True)
            entry = {"ms": round(ms, 4)}
            if flops:
                entry["tflops"] = round(flops / (ms / 1000) / 1e12, 3)
                entry["frac_of_fp32_fma_peak"] = round(flops / (ms / 1000) / 1e12 / fp32_peak, 4)
            if moved:
                entry["gbs"] = round(moved / (ms / 1000) / 1e9, 1)
                entry["frac_of_hbm"] = round(moved / (ms / 1000) / 1e9 / peaks["hbm_gbs"], 4)
            out[key] = entry

        for name, lens in (("prompt", [PREFILL_TOKENS]), ("decode", [1] * batch)):
            tokens = sum(lens)
            cu, slots = dev([0] + [sum(lens[:i + 1]) for i in range(len(lens))]), dev(list(range(len(lens))))
            rand = lambda *shape: torch.randn(shape, device=device, generator=g)
            scan_flops = 5.0 * tokens * H * D * V
            # retention: float32 rows [q | k | v] made by rotary_rows, then the scan with a constant decay
            x = rand(tokens, 2 * H * D + 2 * H * V).to(torch.bfloat16)
            positions = dev([i for n in lens for i in range(PROMPT_LEN, PROMPT_LEN + n)])
            freq = (1000000.0 ** (-torch.arange(0, D, 2, device=device).float() / D)).contiguous()
            record(f"{name}_rotary_rows", lambda: ops.rotary_rows(x, positions, freq, num_heads=H, head_dim=D, v_dim=V,
                                                                  rotary_dims=D, q_off=0, k_off=H * D, v_off=2 * H * D,
                                                                  k_scale=D ** -0.5),
                   moved=tokens * (2.0 + 4.0) * (2 * H * D + H * V))
            rows = ops.rotary_rows(x, positions, freq, num_heads=H, head_dim=D, v_dim=V, rotary_dims=D, q_off=0,
                                   k_off=H * D, v_off=2 * H * D, k_scale=D ** -0.5)
            kw = dict(num_heads=H, head_dim=D, v_dim=V, q_off=0, k_off=H * D, v_off=2 * H * D)
            record(f"{name}_retention_scan", lambda: ops.linear_scan(rows, state, cu, slots, mode="plain_decay",
                                                                     decay=decay, **kw),
                   flops=scan_flops, moved=2.0 * 4 * len(lens) * floats + 4.0 * tokens * (2 * H * D + 2 * H * V))
            record(f"{name}_like_lightning_scan", lambda: ops.linear_scan(x, state, cu, slots, mode="constant_decay",
                                                                          decay=decay, **kw),
                   flops=scan_flops, moved=2.0 * 4 * len(lens) * floats + 2.0 * tokens * 3 * H * D + 4.0 * tokens * H * V)
            o = ops.linear_scan(rows, state, cu, slots, mode="plain_decay", decay=decay, **kw)
            record(f"{name}_norm_per_head_silu_gate", lambda: ops.group_norm_gate(
                o, None, group=V, eps=1e-6, out_dtype=torch.bfloat16, x=x, gate_off=2 * H * D + H * V, gate="silu"),
                moved=8.0 * tokens * H * V)
            norm_wide = torch.ones((H * V,), device=device)
            record(f"{name}_like_norm_all_heads_gated", lambda: ops.group_norm_gate(
                o, norm_wide, group=H * V, eps=1e-6, out_dtype=torch.bfloat16, x=x, gate_off=2 * H * D + H * V),
                moved=8.0 * tokens * H * V)
            # the state-space mixer: preparation, the scan with a decay per token (all heads on one q and k), the norm
            xin = rand(tokens, 2 * H * V + 2 * D + H).to(torch.bfloat16)
            conv, bias = torch.rand((channels, taps), device=device, generator=g) - 0.3, torch.zeros((channels,), device=device)
            step_bias, rate_log = torch.full((H,), -3.0, device=device), torch.zeros((H,), device=device)
            state.zero_()
            prep_kw = dict(tail_off=floats, num_heads=H, v_dim=V, state_dim=D, groups=1, taps=taps, conv_off=H * V,
                           step_off=H * V + channels)
            width = ops.ssm_prep_width(H, V, D, 1)
            record(f"{name}_ssm_prep", lambda: ops.ssm_prep(xin, conv, bias, step_bias, rate_log, state, cu, slots, **prep_kw),
                   moved=tokens * (2.0 * (channels + H) + 4.0 * width))
            prepared = ops.ssm_prep(xin, conv, bias, step_bias, rate_log, state, cu, slots, **prep_kw)
            record(f"{name}_ssm_scan", lambda: ops.linear_scan(
                prepared, state, cu, slots, num_heads=H, head_dim=D, v_dim=V, mode="token_decay", q_off=0, k_off=D,
                v_off=2 * D, qk_group=H, decay_off=2 * D + H * V),
                flops=scan_flops, moved=2.0 * 4 * len(lens) * floats + 4.0 * tokens * (2 * D + 2 * H * V + H))
            so = ops.linear_scan(prepared, state, cu, slots, num_heads=H, head_dim=D, v_dim=V, mode="token_decay",
                                 q_off=0, k_off=D, v_off=2 * D, qk_group=H, decay_off=2 * D + H * V)
            skip = torch.ones((H,), device=device)
            record(f"{name}_ssm_norm_skip_gate_first", lambda: ops.group_norm_gate(
                so, norm_wide, group=H * V, eps=1e-6, out_dtype=torch.bfloat16, x=xin, gate_off=0, gate="silu",
                gate_first=True, skip=prepared, skip_off=2 * D + H * V + H, skip_coef=skip, skip_head=V),
                moved=12.0 * tokens * H * V)
            record(f"{name}_conv_tail", lambda: ops.conv_tail(xin, state, cu, slots, tail_off=floats, conv_off=H * V,
                                                              channels=channels, taps=taps))
            # the like kernel: the delta rule's preparation at the same heads and widths
            dch = 2 * kvh * D + H * V
            xd = rand(tokens, dch + H * V + 2 * H).to(torch.bfloat16)
            dconv = torch.rand((dch, taps), device=device, generator=g) - 0.3
            state.zero_()
            record(f"{name}_like_delta_prep", lambda: ops.delta_prep(
                xd, dconv, step_bias, rate_log, state, cu, slots, unit_eps=1e-6, num_heads=H, num_kv_heads=kvh,
                head_dim=D, v_dim=V, taps=taps), moved=tokens * (2.0 * (dch + 2 * H) + 4.0 * (dch + 2 * H)))
            state.zero_()
            # the stream in copies: write + read + norm in one pass, beside the residual add + RMS norm
            streams = rand(tokens, S, W)
            y = rand(tokens, W).to(torch.bfloat16)
            pending = ops.HyperPending(y, torch.eye(S, device=device), torch.ones((S,), device=device),
                                       torch.ones((W,), device=device))
            read, weight = torch.ones((S,), device=device), torch.ones((W,), device=device)
            record(f"{name}_hyper_step", lambda: ops.hyper_step(streams, pending, read, weight, 1e-6, torch.bfloat16),
                   moved=tokens * W * (8.0 * S + 4.0))
            hidden = rand(tokens, W)
            record(f"{name}_like_add_rmsnorm", lambda: ops.add_rmsnorm(hidden, y, weight, 1e-6, torch.bfloat16),
                   moved=tokens * W * 12.0)
            a, b = rand(tokens, W), rand(tokens, W)
            record(f"{name}_normed_pair_sum", lambda: ops.normed_pair_sum(a, b, weight, weight, eps=1e-6, sa=0.5, sb=0.5,
                                                                          out_dtype=torch.float32),
                   moved=tokens * W * 12.0)
            ab, bb = a.to(torch.bfloat16), b.to(torch.bfloat16)
            record(f"{name}_like_scaled_sum", lambda: ops.scaled_sum(ab, bb, 0.5, 0.5), moved=tokens * W * 6.0)
            # the rotation before attention, with and without norms over the whole q and k rows
            bf = dict(dtype=torch.bfloat16, device=device)
            k_pages = torch.zeros((tokens // page + 1, kvh, page, D), **bf)
            v_pages = torch.zeros((tokens // page + 1, kvh, page, D), **bf)
            xp = rand(tokens, (heads + 2 * kvh) * D).to(torch.bfloat16)
            slot_map = dev(list(range(tokens)))
            half = freq[: D // 4].contiguous()
            qn, kn = torch.ones((heads * D,), device=device), torch.ones((kvh * D,), device=device)
            prep = dict(num_heads=heads, num_kv_heads=kvh, head_dim=D, v_dim=D, rotary_dims=D // 2, layout="half")
            moved = 2.0 * tokens * ((heads + 2 * kvh) * D + heads * D + 2 * kvh * D)
            record(f"{name}_rotary_prep_row_norms", lambda: ops.rotary_prep(
                xp, positions, slot_map, half, k_pages, v_pages, q_norm=qn, k_norm=kn, row_norm_eps=1e-6, **prep), moved=moved)
            record(f"{name}_like_rotary_prep", lambda: ops.rotary_prep(xp, positions, slot_map, half, k_pages, v_pages, **prep),
                   moved=moved)
        return out

    sizes = {}
    if design == "zavizen":
        with ClockSampler() as clocks:
            for name, z in RENADRA_SIZES.items():
                sizes[name] = {"zavizen": measure(zavizen_config(z, layers)),
                               "renadra": measure(renadra_config(z, layers)),
                               "kernels": zavizen_kernels_alone(z)}
        head = sizes["4k"]["zavizen"]
        line = {"metric": "decode tok/s at batch 8 of four Zavizen layers (width 4,096, B200); prefill, a smaller size, "
                          "Renadra layers of equal size and Zavizen's kernels alone, each beside the like kernel of "
                          "another design, alongside",
                "value": head["decode_tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": head["decode_ms"], "higher_is_better": True, "dtype": "bf16",
                "data": "synthetic (seeded uniform token ids, seeded random weights)",
                "config": {"model": "Zavizen", "layers": layers, "sizes": RENADRA_SIZES, "streams": ZAVIZEN_STREAMS,
                           "vocab": SUKALORN_VOCAB, "global_batch": batch, "prompt_len": PROMPT_LEN,
                           "prefill_tokens": PREFILL_TOKENS, "page_size": args.page_size,
                           "l2": "whole steps: inputs larger than L2; kernels alone: L2 flushed (a 256 MB write) before "
                                 "every timed launch", "peaks": peaks["source"], "fp32_fma_tflops": FP32_FMA_TFLOPS},
                "gpu_launches": head["launches_per_decode_step"] * args.steps, "sizes": sizes,
                "clocks": clocks.summary()}
        print(json.dumps(line))
        return 0
    if design == "renadra":
        with ClockSampler() as clocks:
            for name, z in RENADRA_SIZES.items():
                sizes[name] = {"renadra": measure(renadra_config(z, layers)),
                               "zifuzen_dense": measure(zifuzen_dense_like(z, layers)),
                               "kernels": renadra_kernels_alone(z)}
        head = sizes["4k"]["renadra"]
        line = {"metric": "decode tok/s at batch 8 of four Renadra layers (width 4,096, B200); prefill, a smaller size, "
                          "Zifuzen layers of equal size with dense feed-forwards and Renadra's kernels alone, each "
                          "beside the like kernel of another design, alongside",
                "value": head["decode_tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": head["decode_ms"], "higher_is_better": True, "dtype": "bf16",
                "data": "synthetic (seeded uniform token ids, seeded random weights)",
                "config": {"model": "Renadra", "layers": layers, "sizes": RENADRA_SIZES, "vocab": SUKALORN_VOCAB,
                           "global_batch": batch, "prompt_len": PROMPT_LEN, "prefill_tokens": PREFILL_TOKENS,
                           "page_size": args.page_size, "l2": "whole steps: inputs larger than L2; kernels alone: L2 "
                           "flushed (a 256 MB write) before every timed launch", "peaks": peaks["source"],
                           "fp32_fma_tflops": FP32_FMA_TFLOPS},
                "gpu_launches": head["launches_per_decode_step"] * args.steps, "sizes": sizes,
                "clocks": clocks.summary()}
        print(json.dumps(line))
        return 0
    if design == "zifuzen":
        with ClockSampler() as clocks:
            for name, z in ZIFUZEN_SIZES.items():
                sizes[name] = {"zifuzen": measure(zifuzen_config(z, layers)), "qwen3": measure(qwen3_like(z, layers)),
                               "kernels": zifuzen_kernels_alone(z)}
        head = sizes["4k"]["zifuzen"]
        line = {"metric": "decode tok/s at batch 8 of four Zifuzen layers (width 4,096, B200); prefill, a smaller size, "
                          "Qwen3 layers of equal size and the delta-rule and routed-expert kernels alone alongside",
                "value": head["decode_tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": head["decode_ms"], "higher_is_better": True, "dtype": "bf16",
                "data": "synthetic (seeded uniform token ids, seeded random weights)",
                "config": {"model": "Zifuzen", "layers": layers, "sizes": ZIFUZEN_SIZES, "vocab": SUKALORN_VOCAB,
                           "global_batch": batch, "prompt_len": PROMPT_LEN, "prefill_tokens": PREFILL_TOKENS,
                           "page_size": args.page_size, "l2": "whole steps: inputs larger than L2; kernels alone: L2 "
                           "flushed (a 256 MB write) before every timed launch", "peaks": peaks["source"],
                           "fp32_fma_tflops": FP32_FMA_TFLOPS},
                "gpu_launches": head["launches_per_decode_step"] * args.steps, "sizes": sizes,
                "clocks": clocks.summary()}
        print(json.dumps(line))
        return 0
    with ClockSampler() as clocks:
        for name, z in SUKALORN_SIZES.items():
            sizes[name] = {"sukalorn": measure(sukalorn_config(z, layers)), "qwen3": measure(qwen3_like(z, layers)),
                           "kernels": kernels_alone(z)}
    head = sizes["4k"]["sukalorn"]
    line = {"metric": "decode tok/s at batch 8 of four Sukalorn layers (width 4,096, B200); prefill, a smaller size, "
                      "Qwen3 layers of equal size and the attention kernels alone alongside",
            "value": head["decode_tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": head["decode_ms"], "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic (seeded uniform token ids, seeded random weights)",
            "config": {"model": "Sukalorn", "layers": layers, "sizes": SUKALORN_SIZES, "vocab": SUKALORN_VOCAB,
                       "global_batch": batch, "prompt_len": PROMPT_LEN, "prefill_tokens": PREFILL_TOKENS,
                       "page_size": args.page_size, "l2": "whole steps: inputs larger than L2; kernels alone: L2 "
                       "flushed (a 256 MB write) before every timed launch", "peaks": peaks["source"]},
            "gpu_launches": head["launches_per_decode_step"] * args.steps, "sizes": sizes, "clocks": clocks.summary()}
    print(json.dumps(line))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens per cache page (a power of two, 16 or more)")
    parser.add_argument("--shape", choices=sorted(SHAPES) + ["renadra", "sukalorn", "zavizen", "zifuzen"], default="8b",
                        help="8b: the headline benchmark; 14b: a mixed scheduler load of 64 requests; 32b: long-context "
                             "decode at batch 16; sukalorn: prefill and decode of the Sukalorn design at two layer "
                             "sizes beside Qwen3 layers of equal size; zifuzen: the same for the Zifuzen design; renadra: the Renadra design beside "
                             "Zifuzen layers of equal size; zavizen: the Zavizen design beside Renadra layers of equal "
                             "size (each prints its own one line)")
    parser.add_argument("--layers", type=int, default=None,
                        help="run fewer layers of the same sizes (reported in config beside the full count)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 decode points")
    args = parser.parse_args()

    if args.shape in ("renadra", "sukalorn", "zavizen", "zifuzen"):
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference arm runs the 8b shape only"}))
            return 0
        if args.gpus != 1:
            print(json.dumps({"error": "this engine runs on one GPU; --gpus must be 1", "n_gpus": args.gpus}))
            return 2
        args.warmup = max(3, args.warmup)
        return sukalorn_shape(args, design=args.shape)
    if args.layers is None:
        args.layers = SHAPES[args.shape]["num_hidden_layers"]
    if args.impl == "reference":
        if args.shape != "8b":
            print(json.dumps({"impl": "reference", "unavailable": "the reference arm runs the 8b shape only"}))
            return 0
        if args.gpus != 1:
            print(json.dumps({"impl": "reference", "unavailable": "the reference runs on one GPU; --gpus must be 1"}))
            return 0
        return reference_arm(args)
    if args.gpus != 1:
        print(json.dumps({"error": "this engine runs on one GPU; --gpus must be 1", "n_gpus": args.gpus}))
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.shape == "14b":
        return serving_shape(args)
    if args.shape == "32b":
        return long_context_shape(args)

    import torch
    from ampere_kv_engine_b200.engine.batch import SeqStep
    from ampere_kv_engine_b200.engine.engine import Engine
    from ampere_kv_engine_b200.kernels import ops
    from ampere_kv_engine_b200.sampling.sampler import SamplingParams

    cfg = dict(QWEN3_8B)
    cfg["num_hidden_layers"] = args.layers
    peaks = load_peaks()
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    max_batch = 64 if not args.no_points else args.batch
    pool_tokens = max(max_batch * (PROMPT_LEN + GEN_LEN + 64),
                      max(args.batch * (CONTEXT + 64), SERVING_REQUESTS * (SERVING_PROMPT[1] + SERVING_OUTPUT[1]) // 2
                          + SERVING_REQUESTS * 64) if not args.no_points else 0,
                      PREFILL_TOKENS + 64)
    from ampere_kv_engine_b200.config.engine_config import EngineConfig
    engine = Engine.from_random(cfg, seed=0, device=device, config=EngineConfig(
        dtype="bfloat16", page_size=args.page_size, max_tokens=pool_tokens, max_seqs=max_batch + 2,
        max_batch_tokens=PREFILL_TOKENS, max_context=CONTEXT))
    runner = engine.runner
    gen = torch.Generator().manual_seed(1234)
    vocab = cfg["vocab_size"]

    def synthetic(n):
        return torch.randint(0, vocab, (n,), generator=gen).tolist()

    def timed(fn, steps):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / steps

    def decode_point(batch, steps, warmup, prompt_len=PROMPT_LEN):
        """ms per decode step of ``batch`` requests that each hold a ``prompt_len``-token prompt."""
        seqs = [runner.open(f"d{batch}-{prompt_len}-{i}") for i in range(batch)]
        if prompt_len <= PREFILL_TOKENS:
            per_step = max(1, PREFILL_TOKENS // prompt_len)
            for i in range(0, batch, per_step):
                runner.step([SeqStep(s, synthetic(prompt_len), []) for s in seqs[i:i + per_step]])
        else:
            for s in seqs:       # long prompts go in portions of the prefill budget
                for start in range(0, prompt_len, PREFILL_TOKENS):
                    runner.step([SeqStep(s, synthetic(min(PREFILL_TOKENS, prompt_len - start)), [])])
        greedy = [SamplingParams()] * batch
        zeros = [0] * batch

        def one():
            logits = runner.step([SeqStep(s, [t], [0]) for s, t in zip(seqs, synthetic(batch))])
            engine.sampler.sample(logits, greedy, zeros)

        for _ in range(warmup):
            one()
        ctx_start = seqs[0].length
        ops.launch_count = 0
        ms = timed(one, steps)
        launches = ops.launch_count
        mean_ctx = ctx_start + (steps + 1) / 2
        runner.raise_on_status()
        for s in seqs:
            runner.close(s)
        return ms, mean_ctx, launches

    with ClockSampler() as clocks:
        ms, mean_ctx, launches = decode_point(args.batch, args.steps, args.warmup)
    clock_summary = clocks.summary()
    value = args.batch / (ms / 1000)
    bytes_step = decode_bytes(cfg, args.layers, args.batch, mean_ctx)
    achieved = bytes_step / (ms / 1000) / 1e9

    # end to end: the scheduler loop of the Python entry point, host tokens in and out every step
    scheduler = engine.new_scheduler()
    slack = args.batch * PROMPT_LEN // PREFILL_TOKENS + 4     # early requests decode while later ones prefill
    requests = [scheduler.submit(f"e{i}", synthetic(PROMPT_LEN), args.warmup + args.steps + slack, ignore_eos=True)
                for i in range(args.batch)]
    while any(not r.output_ids for r in requests):
        scheduler.step()
    for _ in range(args.warmup):
        scheduler.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    stats = None
    for _ in range(args.steps):
        _, stats = scheduler.step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1000 / args.steps
    assert stats.decode_tokens == args.batch and stats.prefill_tokens == 0
    for r in requests:
        scheduler.cancel(r)
    scheduler.step()
    h2d = runner.last_h2d_bytes + 8 * args.batch      # the step's index buffer + temperatures and uniforms
    e2e = {"value": round(args.batch / (e2e_ms / 1000), 2), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * (args.batch + 1)}

    # prefill of 2,048 tokens in one step
    def prefill_once():
        seq = runner.open("prefill")
        logits = runner.step([SeqStep(seq, prompt, [PREFILL_TOKENS - 1])])
        engine.sampler.sample(logits, [SamplingParams()], [0])
        runner.close(seq)

    prompt = synthetic(PREFILL_TOKENS)
    for _ in range(3):
        prefill_once()
    prefill_ms = timed(prefill_once, 5)
    flops = prefill_flops(cfg, args.layers, PREFILL_TOKENS)
    prefill = {"value": round(PREFILL_TOKENS / (prefill_ms / 1000), 1), "tokens": PREFILL_TOKENS,
               "ms": round(prefill_ms, 3),
               "frac": round(flops["gemm"] / (prefill_ms / 1000) / (peaks["bf16_tflops"] * 1e12), 4),
               "frac_of": "matrix-product FLOPs / burst bf16 peak", "gemm_tflop": round(flops["gemm"] / 1e12, 3),
               "attention_tflop": round(flops["attention"] / 1e12, 3),
               "frac_with_attention": round((flops["gemm"] + flops["attention"]) / (prefill_ms / 1000)
                                            / (peaks["bf16_tflops"] * 1e12), 4)}

    points = {}
    if not args.no_points:
        for b in (1, 64):
            p_ms, _, _ = decode_point(b, max(8, args.steps // 2), args.warmup)
            points[f"decode_b{b}"] = round(b / (p_ms / 1000), 2)
        # the same batch at the end of the configuration's 8,192-token context, with its own roofline fraction
        long_steps = max(8, args.steps // 2)
        p_ms, long_ctx, _ = decode_point(args.batch, long_steps, args.warmup, CONTEXT - GEN_LEN)
        points[f"decode_b{args.batch}_ctx{CONTEXT}"] = round(args.batch / (p_ms / 1000), 2)
        points[f"decode_b{args.batch}_ctx{CONTEXT}_hbm_frac"] = round(
            decode_bytes(cfg, args.layers, args.batch, long_ctx) / (p_ms / 1000) / 1e9 / peaks["hbm_gbs"], 4)
        # a scheduler load: many requests of mixed lengths, chunked prefill beside decoding, host tokens in and out
        # (second pass timed: the decode graphs of its batch sizes exist by then); tokens per second of wall clock
        serving = serving_load(engine, synthetic, SERVING_REQUESTS, SERVING_PROMPT, SERVING_OUTPUT)
        points.update(serving)
        # a prompt arrives while the batch decodes: what the newcomer waits for its first token and what the
        # running requests feel meanwhile (the figures of the reference's scheduler benchmark,
        # ampere_kv/bench_scheduler.py:115-125, 242-271)
        points.update(insert_point(engine, synthetic, args.batch))

    line = {
        "metric": "decode tok/s at batch 8 (Qwen3-8B shape, B200); prefill and batch 1/64 alongside",
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded uniform token ids, seeded random weights)",
        "config": {
            "model": "Qwen3-8B shape", "layers": args.layers, "layers_full": QWEN3_8B["num_hidden_layers"],
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": vocab,
            "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "gen_len": GEN_LEN,
            "mean_decode_context": round(mean_ctx, 1), "page_size": args.page_size, "kv_dtype": "bf16",
            "parallelism": "single GPU", "l2": "inputs larger than L2 (all weights stream every step)",
        },
        "e2e": e2e,
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "peaks": peaks["source"]},
        "points": points,
        "clocks": clock_summary,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
