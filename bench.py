"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]

The default run has the layer sizes of Qwen2.5-1.5B (28 layers, hidden 1536, 12 query / 2 KV heads of
128, feed-forward 8960, vocabulary 151936, tied head) with random bfloat16 weights, a batch of 8
requests with 1,024-token prompts, and times K decode steps (one new token per request per step).
It prints ONE JSON line:

* ``value``: decoded tokens per second, device-timed (CUDA events around the K steps);
* ``e2e``: the same through ``LLMEngine.step()``: token ids from host memory in, sampled ids back to
  the host, every step;
* ``prefill``: one 2,048-token prompt in one step (tokens/s, ms, fraction of the bf16 matrix peak);
* ``roofline``: bytes the decode step must read (every weight once + the KV of the live requests)
  divided by its time, against the measured copy bandwidth;
* ``points``: decode at batch 1 and 64.

Weights (3.1 GB) are far larger than the 126 MB L2, so every step streams them from HBM; no L2 flush
is needed between iterations.  Peaks come from MEASURED_PEAKS.json when the driver wrote it, else from
the fallback figures of an earlier measurement on this pool (6.65 TB/s copy, 1.59 PFLOP/s bf16).
"""

from __future__ import annotations

import argparse
import json
import os
import random
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT_LEN = 1024
GENERATED = 256
PREFILL_LEN = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            out = dict(FALLBACK_PEAKS)
            for key in out:
                if key in data and isinstance(data[key], (int, float)):
                    out[key] = float(data[key])
            return out, "measured"
        except (json.JSONDecodeError, OSError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi in the background during the timed region (reads settings only)."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20", "-i", "0"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def lines(self) -> int:
        try:
            return len(Path(self.file.name).read_text().splitlines())
        except OSError:
            return 0

    def mark(self) -> None:
        """What was sampled so far (the tool takes a moment to start) is not of the timed region."""
        self.skip = self.lines()

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        try:
            for line in Path(self.file.name).read_text().splitlines()[getattr(self, "skip", 0):]:
                cols = [c.strip() for c in line.split(",")]
                if len(cols) < 9:
                    continue
                try:
                    sm.append(float(cols[1]))
                    mx.append(float(cols[2]))
                except ValueError:
                    continue
                for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                    if cols[col].lower().startswith("active"):
                        reasons.add(name)
        finally:
            try:
                os.unlink(self.file.name)
            except OSError:
                pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm() -> int:
    # `pip install --no-index --no-build-isolation --find-links /opt/wheelhouse --target baseline/_ref`
    # of the reference fails: its build backend (hatchling) is not in the offline wheelhouse.
    ref = ROOT / "baseline" / "_ref" / "clockwork"
    if not ref.is_dir():
        print(json.dumps({"impl": "reference", "unavailable":
                          "reference not installed: pip cannot build it offline (build backend hatchling is missing from the wheelhouse)"}))
        return 0
    print(json.dumps({"impl": "reference", "unavailable": "reference arm not wired: no offline install was possible when this was written"}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (reported in config)")
    ap.add_argument("--shape", default="qwen2.5-1.5b")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 / 64 and prefill (quick runs)")
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="run one part only and print its figures (for profiling runs under ncu)")
    ap.add_argument("--timeline", action="store_true",
                    help="with --only decode: also print one step's kernel timeline (device-side records, ops/trace.py)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch

    from clockwork_b200 import EngineConfig
    from clockwork_b200.cli import SHAPES, shape_config
    from clockwork_b200.engine import LLMEngine, StepEntry, random_model
    from clockwork_b200.ops.library import launch_count
    from clockwork_b200.sampling import SamplingParams

    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    torch.cuda.set_device(0)
    raw = shape_config(args.shape, args.layers)
    full_layers = SHAPES[args.shape]["num_hidden_layers"]
    model = random_model(raw, seed=0, dtype="bfloat16", device="cuda:0")
    vocab = raw["vocab_size"]
    rng = random.Random(0)
    peak, peak_kind = peaks()

    def make_engine(batch: int) -> LLMEngine:
        page = 16
        tokens_per_seq = PROMPT_LEN + max(GENERATED, 2 * (args.steps + args.warmup)) + 2 * page
        num_blocks = max(batch * ((tokens_per_seq + page - 1) // page) + 8, (PREFILL_LEN + page) // page + 8)
        cfg = EngineConfig.defaults("random", dtype="bfloat16", block_size=page, num_blocks=num_blocks,
                                    max_model_len=4096, max_num_seqs=max(batch, 1), max_num_batched_tokens=4096,
                                    enable_prefix_cache=False, watermark=0.0)
        return LLMEngine(cfg, model=model)

    def fill(engine: LLMEngine, batch: int) -> None:
        """Admit ``batch`` requests with PROMPT_LEN-token prompts and run their prefill."""
        params = SamplingParams(max_tokens=4 * (args.steps + args.warmup) + GENERATED, ignore_eos=True)
        for i in range(batch):
            engine.add_request(f"b{i}", prompt_token_ids=[rng.randrange(vocab) for _ in range(PROMPT_LEN)], sampling_params=params)
        while any(s.num_uncomputed_tokens() > 1 for s in engine.scheduler.running) or engine.scheduler.waiting:
            engine.step()

    def drain(engine: LLMEngine) -> None:
        for rid in [s.seq_id for s in engine.scheduler.running + engine.scheduler.waiting]:
            engine.abort_request(rid)

    def time_decode(batch: int, steps: int, warmup: int) -> dict:
        """Device time of ``steps`` decode steps through the step function, and the end-to-end
        time through LLMEngine.step()."""
        engine = make_engine(batch)
        fill(engine, batch)
        runner, cache = engine.runner, engine.cache
        ids = [s.seq_id for s in engine.scheduler.running]
        assert len(ids) == batch
        ctx_start = cache.get(ids[0]).num_computed
        # ---- end to end: the engine's own loop, host tokens in and out -------------------------------
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        l0 = launch_count() + runner.graph_kernel_launches
        t0 = time.perf_counter()
        for _ in range(steps):
            outs = engine.step()
            assert len(outs) == batch
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        e2e_launches = launch_count() + runner.graph_kernel_launches - l0
        h2d = engine.runner.last_upload_bytes
        # ---- device-timed: the same steps enqueued back to back ---------------------------------------
        tokens = [[rng.randrange(vocab)] for _ in range(batch)]
        ctx_now = cache.get(ids[0]).num_computed
        step_fn = engine.decode_step_device
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler() as clocks:
            # the sampler takes a moment to start reporting: wait for its first line (two seconds at most)
            waited = time.perf_counter()
            while clocks.proc is not None and clocks.lines() == 0 and time.perf_counter() - waited < 2.0:
                time.sleep(0.01)
            for _ in range(warmup):
                step_fn(ids, tokens)
            torch.cuda.synchronize()
            clocks.mark()
            l0 = launch_count() + runner.graph_kernel_launches
            start.record()
            for _ in range(steps):
                step_fn(ids, tokens)
            end.record()
            torch.cuda.synchronize()
        dev_ms = start.elapsed_time(end)
        launches = launch_count() + runner.graph_kernel_launches - l0
        runner.check_status()
        if args.timeline:
            print_timeline(step_fn, ids, tokens)
        ctx_mid = ctx_now + warmup + steps // 2
        kv_bytes = batch * ctx_mid * cache.bytes_per_token()
        result = {
            "batch": batch, "steps": steps, "ms_per_step": dev_ms / steps, "tok_s": batch * steps / (dev_ms / 1e3),
            "e2e_tok_s": batch * steps / e2e_s, "e2e_ms_per_step": e2e_s * 1e3 / steps, "launches": launches,
            "e2e_launches": e2e_launches, "h2d_bytes": h2d, "d2h_bytes": batch * 4 + 16, "ctx_start": ctx_start,
            "ctx_mid": ctx_mid, "bytes": model.weight_bytes() + kv_bytes, "clocks": clocks.summary(),
        }
        drain(engine)
        del engine
        torch.cuda.empty_cache()
        return result

    def print_timeline(step_fn, ids, tokens) -> None:
        """One decode step, kernel by kernel: when the first and last CTA started, when the wait on the
        preceding kernel returned, and when the last CTA was done (microseconds from the step's start)."""
        from clockwork_b200.ops import trace

        trace.enable()
        step_fn(ids, tokens)
        trace.reset()
        step_fn(ids, tokens)
        launches = trace.collect()
        trace.disable()
        print(f"# timeline of one decode step: {len(launches)} traced launches (matrix products and decode attention)")
        print("# grid            ctas   start first..last     released first..last   end first..last   (us)")
        for l in launches:
            f = lambda key: l.get(key, 0) / 1000.0  # noqa: E731
            print(f"# {str(l['grid']):15s} {l['ctas']:4d}  {f('start_first'):9.2f}..{f('start_last'):9.2f}  "
                  f"{f('released_first'):9.2f}..{f('released_last'):9.2f}  {f('end_first'):9.2f}..{f('end_last'):9.2f}")

    def time_prefill(reps: int = 3) -> dict:
        engine = make_engine(1)
        runner, cache = engine.runner, engine.cache
        times = []
        for rep in range(reps + 2):
            rid = f"p{rep}"
            cache.open(rid)
            toks = [rng.randrange(vocab) for _ in range(PREFILL_LEN)]
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            logits = runner.step([StepEntry(rid, toks, [PREFILL_LEN - 1])])
            end.record()
            torch.cuda.synchronize()
            assert logits.shape == (1, vocab)
            if rep >= 2:
                times.append(start.elapsed_time(end))
            cache.close(rid)
        runner.check_status()
        ms = statistics.median(times)
        spec = model.spec
        attn = spec.layers[0].mixer
        h, nh, nkv, hd = spec.hidden_size, attn["num_heads"], attn["num_kv_heads"], attn["head_dim"]
        inter = spec.layers[0].ffn["intermediate_size"]
        per_layer = h * (nh + 2 * nkv) * hd + nh * hd * h + 3 * h * inter
        matrix_flops = 2 * per_layer * len(spec.layers) * PREFILL_LEN + 2 * h * vocab  # one logits row
        attn_flops = len(spec.layers) * 4 * nh * hd * PREFILL_LEN * (PREFILL_LEN + 1) / 2
        flops = matrix_flops + attn_flops
        del engine
        torch.cuda.empty_cache()
        return {"value": PREFILL_LEN / (ms / 1e3), "tokens": PREFILL_LEN, "ms": ms,
                "frac": flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12), "tflops": flops / (ms / 1e3) / 1e12}

    if args.only == "prefill":
        print(json.dumps({"impl": "ours", "prefill": time_prefill(reps=1)}))
        return 0
    main_run = time_decode(args.batch, args.steps, args.warmup)
    if args.only == "decode":
        print(json.dumps({"impl": "ours", "batch": args.batch, "ms_per_step": main_run["ms_per_step"],
                          "tok_s": main_run["tok_s"], "e2e_tok_s": main_run["e2e_tok_s"], "launches": main_run["launches"]}))
        return 0
    out = {
        "metric": "decode tokens/s (Qwen2.5-1.5B shape, random weights)",
        "value": main_run["tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": main_run["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": args.shape, "layers": raw["num_hidden_layers"], "layers_full": full_layers,
            "hidden": raw["hidden_size"], "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
            "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"], "vocab": vocab,
            "tied_head": raw["tie_word_embeddings"], "global_batch": args.batch, "seq_len": PROMPT_LEN + GENERATED,
            "prompt_len": PROMPT_LEN, "context_at_timing": main_run["ctx_mid"], "page_size": 16,
            "parallelism": "single GPU", "l2_policy": "inputs (3.1 GB of weights per step) exceed the 126 MB L2",
            "peaks": peak_kind,
        },
        "clocks": main_run["clocks"],
        "e2e": {"value": main_run["e2e_tok_s"], "unit": "tok/s", "ms_per_step": main_run["e2e_ms_per_step"],
                "h2d_bytes_per_step": main_run["h2d_bytes"], "d2h_bytes_per_step": main_run["d2h_bytes"]},
        "gpu_launches": main_run["launches"],
        "roofline": {"bound": "hbm", "achieved": main_run["bytes"] / (main_run["ms_per_step"] / 1e3) / 1e9,
                     "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": main_run["bytes"] / (main_run["ms_per_step"] / 1e3) / 1e9 / peak["hbm_gbs"],
                     "bytes_per_step": main_run["bytes"], "of": peak_kind},
    }
    if not args.skip_points:
        out["prefill"] = time_prefill()
        points = {}
        for batch in (1, 64):
            r = time_decode(batch, max(16, args.steps // 2), args.warmup)
            points[f"decode_b{batch}"] = r["tok_s"]
            points[f"decode_b{batch}_e2e"] = r["e2e_tok_s"]
            points[f"decode_b{batch}_hbm_frac"] = r["bytes"] / (r["ms_per_step"] / 1e3) / 1e9 / peak["hbm_gbs"]
        out["points"] = points
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
