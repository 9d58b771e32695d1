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
* ``points``: decode at batch 1 and 64, decode at batch 8 over the whole span of contexts 1,024 to
  1,280, a mixed step (32 single tokens at context 2,048 beside two 512-token prompt portions), and
  64 requests that share a 1,536-token prefix through the prefix cache.

A region of K steps is short (26 ms at 20 steps), so it is repeated, each time on freshly prefilled
requests at the same contexts, until the repeats cover a second or so; the median repeat is reported
and the spread is in ``repeats``.  Weights (3.1 GB) are far larger than the 126 MB L2, so every step
streams them from HBM; no L2 flush is needed between iterations.  Peaks come from MEASURED_PEAKS.json
when the driver wrote it, else from the fallback figures of an earlier measurement on this pool
(6.65 TB/s copy, 1.59 PFLOP/s bf16).

``--impl reference`` times the unmodified reference engine (its ``LLMEngine`` over its own
``Qwen2ForCausalLM``, random weights filled in place) on the same shape, batch, prompt length, steps
and warm-up and prints the same line with ``"impl": "reference"``; nothing of this package is imported
on that path.
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
PAGE = 16
MAX_MODEL_LEN = 4096
TARGET_TIMED_S = 1.0  # repeats of the timed region go on until they cover this much
MAX_REPEATS = 48
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# The shape both arms run (the reference arm may import nothing of this package, so the sizes stand
# here too; the engine's own arm checks them against the shape its architecture registers).
QWEN25_1P5B = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=28, hidden_size=1536,
    num_attention_heads=12, num_key_value_heads=2, head_dim=128, intermediate_size=8960, vocab_size=151936,
    rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=32768,
    hidden_act="silu", use_sliding_window=False,
)


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
    """nvidia-smi in the background during the timed region (reads settings only).  The GPU is named
    by the UUID of CUDA device 0 of this process, so that the samples are of the GPU the bench runs
    on whatever CUDA_VISIBLE_DEVICES maps it to."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        self.skip = 0
        self.gpu = self._gpu_id()

    @staticmethod
    def _gpu_id() -> str:
        try:
            import torch

            uuid = str(torch.cuda.get_device_properties(0).uuid)
            return uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:  # noqa: BLE001  (an older torch without the property: the first visible GPU)
            first = os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0].strip()
            return first or "0"

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20", "-i", self.gpu],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def lines(self) -> int:
        try:
            return len(Path(self.file.name).read_text().splitlines())
        except OSError:
            return 0

    def wait_for_first_line(self) -> None:
        """The tool takes a moment to start reporting (two seconds at most are waited for)."""
        waited = time.perf_counter()
        while self.proc is not None and self.lines() == 0 and time.perf_counter() - waited < 2.0:
            time.sleep(0.01)

    def mark(self) -> None:
        """What was sampled so far is not of the timed region."""
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
            for line in Path(self.file.name).read_text().splitlines()[self.skip:]:
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
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"], "gpu": self.gpu}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm),
                "gpu": self.gpu}


def spread(values: list[float]) -> dict:
    return {"n": len(values), "median": statistics.median(values), "min": min(values), "max": max(values)}


def prefill_flops(shape: dict, tokens: int) -> float:
    h, nh, nkv, hd = shape["hidden_size"], shape["num_attention_heads"], shape["num_key_value_heads"], shape["head_dim"]
    per_layer = h * (nh + 2 * nkv) * hd + nh * hd * h + 3 * h * shape["intermediate_size"]
    matrix = 2 * per_layer * shape["num_hidden_layers"] * tokens + 2 * h * shape["vocab_size"]  # one logits row
    attention = shape["num_hidden_layers"] * 4 * nh * hd * tokens * (tokens + 1) / 2
    return matrix + attention


def config_record(shape: dict, full_layers: int, batch: int, ctx: int, peak_kind: str) -> dict:
    return {
        "model": "qwen2.5-1.5b", "layers": shape["num_hidden_layers"], "layers_full": full_layers,
        "hidden": shape["hidden_size"], "heads": shape["num_attention_heads"], "kv_heads": shape["num_key_value_heads"],
        "head_dim": shape["head_dim"], "intermediate": shape["intermediate_size"], "vocab": shape["vocab_size"],
        "tied_head": shape["tie_word_embeddings"], "global_batch": batch, "seq_len": PROMPT_LEN + GENERATED,
        "prompt_len": PROMPT_LEN, "context_at_timing": ctx, "page_size": PAGE, "parallelism": "single GPU",
        "l2_policy": "inputs (3.1 GB of weights per step) exceed the 126 MB L2", "peaks": peak_kind,
    }


# ---------------------------------------------------------------------------------------------------
# the reference arm
# ---------------------------------------------------------------------------------------------------
def find_reference() -> Path | None:
    """The folder that holds the reference's ``clockwork`` package: the copy under baseline/_ref, else a
    checkout named by CLOCKWORK_REFERENCE or lying beside this repository."""
    named = os.environ.get("CLOCKWORK_REFERENCE")
    for base in (ROOT / "baseline" / "_ref", Path(named) if named else None, ROOT.parent / "reference"):
        if base is not None and (base / "clockwork" / "engine" / "llm_engine.py").is_file():
            return base
    return None


def reference_arm(args) -> int:
    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
        return 0

    base = find_reference()
    if base is None:
        return unavailable("the reference's package was found neither under baseline/_ref nor in a checkout beside this repository")
    sys.path.insert(0, str(base))
    try:
        import torch
        from types import SimpleNamespace

        from clockwork.config import EngineConfig
        from clockwork.engine.llm_engine import LLMEngine
        from clockwork.engine.model import Qwen2ForCausalLM
        from clockwork.engine.sequence import SamplingParams
        from clockwork.kernels.attention import resolve_backend
    except Exception as exc:  # noqa: BLE001
        return unavailable(f"importing the reference failed: {type(exc).__name__}: {exc}")
    if not torch.cuda.is_available():
        return unavailable("no CUDA device")
    if args.gpus != 1:
        print(f"bench.py: the reference engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(args.warmup, 3)
    shape = dict(QWEN25_1P5B)
    if args.layers is not None:
        shape["num_hidden_layers"] = args.layers
    hf_config = SimpleNamespace(**shape)
    vocab = shape["vocab_size"]
    rng = random.Random(0)
    peak, peak_kind = peaks()

    class IntTokenizer:
        """Token id <-> decimal string, as the reference's own engine tests use (tests/test_llm_engine.py:17-27)."""
        eos_token_id = None

        def encode(self, text):
            return [int(part) for part in text.split()]

        def decode(self, ids, skip_special_tokens=True):
            return " ".join(str(i) for i in ids)

    try:
        backend = resolve_backend("auto")
        torch.manual_seed(0)
        with torch.device("cuda"):  # build on the GPU: 1.5 G parameters take long to initialise on the host
            model = Qwen2ForCausalLM(hf_config, attention_backend=backend)
        model = model.to(dtype=torch.bfloat16)
        with torch.no_grad():
            for name, p in model.named_parameters():
                if name.endswith("norm.weight") or "layernorm" in name:
                    p.normal_(0.0, 0.1).add_(1.0)
                else:
                    p.normal_(0.0, 0.02)

        def make_engine(batch: int, steps: int):
            tokens_per_seq = PROMPT_LEN + 2 * (steps + warmup) + 2 * PAGE
            num_blocks = max(batch * ((tokens_per_seq + PAGE - 1) // PAGE) + 8, (PREFILL_LEN + PAGE) // PAGE + 8)
            cfg = EngineConfig.defaults("random", dtype="bfloat16", device="cuda", block_size=PAGE, num_blocks=num_blocks,
                                        max_model_len=MAX_MODEL_LEN, max_num_seqs=max(batch, 1),
                                        max_num_batched_tokens=8192, enable_prefix_cache=False, watermark=0.0,
                                        attention_backend=backend)
            return LLMEngine(cfg, model=model, hf_config=hf_config, tokenizer=IntTokenizer())

        def time_decode(batch: int, steps: int, sampler=None) -> dict:
            """Repeats of: fresh requests prefilled, W untimed steps, K timed steps of the engine's own loop."""
            dev_ms, wall_ms = [], []
            total = 0.0
            ctx = None
            while total < TARGET_TIMED_S and len(dev_ms) < MAX_REPEATS:
                engine = make_engine(batch, steps)
                params = SamplingParams(max_tokens=4 * (steps + warmup) + GENERATED, ignore_eos=True)
                for i in range(batch):
                    engine.add_request(f"b{i}", prompt_token_ids=[rng.randrange(vocab) for _ in range(PROMPT_LEN)], sampling_params=params)
                while engine.scheduler.waiting:
                    engine.step()
                for _ in range(warmup):
                    engine.step()
                ctx = len(engine.scheduler.running[0])
                torch.cuda.synchronize()
                if sampler is not None and not dev_ms:
                    sampler.mark()
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0 = time.perf_counter()
                start.record()
                for _ in range(steps):
                    outs = engine.step()
                    assert len(outs) == batch
                end.record()
                torch.cuda.synchronize()
                wall = time.perf_counter() - t0
                dev_ms.append(start.elapsed_time(end) / steps)
                wall_ms.append(wall * 1e3 / steps)
                total += wall
                for i in range(batch):
                    engine.abort_request(f"b{i}")
                del engine
            return {"ms": statistics.median(dev_ms), "e2e_ms": statistics.median(wall_ms), "repeats": spread(dev_ms),
                    "ctx": ctx + steps // 2}

        def time_prefill(reps: int = 3) -> dict:
            times = []
            for rep in range(reps + 2):
                engine = make_engine(1, 1)
                engine.add_request("p", prompt_token_ids=[rng.randrange(vocab) for _ in range(PREFILL_LEN)],
                                   sampling_params=SamplingParams(max_tokens=2, ignore_eos=True))
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                start.record()
                outs = engine.step()
                end.record()
                torch.cuda.synchronize()
                assert len(outs) == 1
                if rep >= 2:
                    times.append(start.elapsed_time(end))
                engine.abort_request("p")
                del engine
            ms = statistics.median(times)
            flops = prefill_flops(shape, PREFILL_LEN)
            return {"value": PREFILL_LEN / (ms / 1e3), "tokens": PREFILL_LEN, "ms": ms,
                    "frac": flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12), "tflops": flops / (ms / 1e3) / 1e12}

        with ClockSampler() as clocks:
            clocks.wait_for_first_line()
            main_run = time_decode(args.batch, args.steps, clocks)
        weight_bytes = sum(p.numel() * p.element_size() for p in model.parameters())
        kv_per_token = shape["num_hidden_layers"] * 2 * shape["num_key_value_heads"] * shape["head_dim"] * 2
        step_bytes = weight_bytes + args.batch * main_run["ctx"] * kv_per_token
        out = {
            "metric": "decode tokens/s (Qwen2.5-1.5B shape, random weights)",
            "value": args.batch / (main_run["ms"] / 1e3), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
            "ms_per_step": main_run["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "impl": "reference", "attention_backend": backend,
            "config": config_record(shape, QWEN25_1P5B["num_hidden_layers"], args.batch, main_run["ctx"], peak_kind),
            "clocks": clocks.summary(), "repeats": main_run["repeats"],
            "e2e": {"value": args.batch / (main_run["e2e_ms"] / 1e3), "unit": "tok/s", "ms_per_step": main_run["e2e_ms"],
                    "h2d_bytes_per_step": None, "d2h_bytes_per_step": None},
            "roofline": {"bound": "hbm", "achieved": step_bytes / (main_run["ms"] / 1e3) / 1e9, "peak": peak["hbm_gbs"],
                         "unit": "GB/s", "frac": step_bytes / (main_run["ms"] / 1e3) / 1e9 / peak["hbm_gbs"],
                         "bytes_per_step": step_bytes, "of": peak_kind},
        }
        if not args.skip_points:
            out["prefill"] = time_prefill()
            points = {}
            for batch in (1, 64):
                r = time_decode(batch, max(16, args.steps // 2))
                points[f"decode_b{batch}"] = batch / (r["ms"] / 1e3)
                points[f"decode_b{batch}_e2e"] = batch / (r["e2e_ms"] / 1e3)
            out["points"] = points
    except Exception as exc:  # noqa: BLE001
        return unavailable(f"the reference failed at the 1.5B shape on this box: {type(exc).__name__}: {exc}")
    print(json.dumps(out))
    return 0


# ---------------------------------------------------------------------------------------------------
# this engine's arm
# ---------------------------------------------------------------------------------------------------
def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--temperature", type=float, default=0.0,
                    help="with --only decode: the requests sample with this temperature (and --top-k, --top-p) in the end-to-end "
                         "steps; the device-timed steps stay greedy")
    ap.add_argument("--top-k", type=int, default=-1)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (reported in config)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="qwen2.5-1.5b",
                    help="with --only: another size that the architecture knows by name (qwen2.5-7b, qwen2.5-32b)")
    ap.add_argument("--skip-points", action="store_true", help="leave out the points and the prefill (quick runs)")
    ap.add_argument("--only", choices=["decode", "prefill", "mixed", "shared-prefix", "long-prompt"], default=None,
                    help="run one part only, once, and print its figures (for profiling runs under ncu)")
    ap.add_argument("--prompt-len", type=int, default=None,
                    help="with --only decode: prompts of this many tokens instead of 1,024 (decoding at other context "
                         "lengths); with --only prefill: a prompt of this many tokens instead of 2,048; with --only long-prompt: "
                         "a prompt of this many tokens instead of 32,768, in portions of 2,048")
    ap.add_argument("--timeline", action="store_true",
                    help="with --only decode: also print one step's kernel timeline (device-side records, ops/trace.py)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    if (args.temperature != 0.0 or args.top_k != -1 or args.top_p != 1.0) and args.only != "decode":
        print("bench.py: --temperature, --top-k and --top-p go with --only decode")
        return 2
    if args.prompt_len is not None and args.only not in ("decode", "prefill", "long-prompt"):
        print("bench.py: --prompt-len goes with --only decode, --only prefill or --only long-prompt")
        return 2
    if args.shape != "qwen2.5-1.5b" and args.only is None:
        print("bench.py: the benchmark line is that of qwen2.5-1.5b; other shapes run with --only")
        return 2

    import torch

    from clockwork_b200 import EngineConfig
    from clockwork_b200.cli import shape_config
    from clockwork_b200.engine import LLMEngine, StepEntry, random_model
    from clockwork_b200.ops.library import launch_count
    from clockwork_b200.sampling import SamplingParams

    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    torch.cuda.set_device(0)
    raw = shape_config(args.shape, args.layers)
    registered = shape_config("qwen2.5-1.5b")
    assert all(registered[k] == v for k, v in QWEN25_1P5B.items()), "the two arms would not run the same shape"
    full_layers = shape_config(args.shape)["num_hidden_layers"]
    model = random_model(raw, seed=0, dtype="bfloat16", device="cuda:0")
    vocab = raw["vocab_size"]
    rng = random.Random(0)
    peak, peak_kind = peaks()
    once = args.only is not None
    prompt_len = args.prompt_len or PROMPT_LEN

    def make_engine(batch: int, steps: int, **overrides) -> LLMEngine:
        tokens_per_seq = prompt_len + 2 * (steps + args.warmup) + 2 * PAGE
        num_blocks = max(batch * ((tokens_per_seq + PAGE - 1) // PAGE) + 8, (PREFILL_LEN + PAGE) // PAGE + 8)
        settings = dict(dtype="bfloat16", block_size=PAGE, num_blocks=num_blocks, max_model_len=max(MAX_MODEL_LEN, tokens_per_seq),
                        max_num_seqs=max(batch, 1), max_num_batched_tokens=4096, enable_prefix_cache=False, watermark=0.0)
        settings.update(overrides)
        return LLMEngine(EngineConfig.defaults("random", **settings), model=model)

    def fill(engine: LLMEngine, batch: int, steps: int, prompt_len: int = prompt_len) -> list[str]:
        """Admit ``batch`` requests with prompts of ``prompt_len`` tokens and run their prefill."""
        for i in range(batch):
            params = SamplingParams(max_tokens=4 * (steps + args.warmup) + GENERATED, ignore_eos=True, temperature=args.temperature,
                                    top_k=args.top_k, top_p=args.top_p, seed=i if args.temperature > 0 else None)
            engine.add_request(f"b{i}", prompt_token_ids=[rng.randrange(vocab) for _ in range(prompt_len)], sampling_params=params)
        while any(s.num_uncomputed_tokens() > 1 for s in engine.scheduler.running) or engine.scheduler.waiting:
            engine.step()
        return [s.seq_id for s in engine.scheduler.running]

    def drain(engine: LLMEngine) -> None:
        for rid in [s.seq_id for s in engine.scheduler.running + engine.scheduler.waiting]:
            engine.abort_request(rid)

    def time_decode(batch: int, steps: int, warmup: int, sampler: ClockSampler | None = None, target_s: float = TARGET_TIMED_S) -> dict:
        """Repeats of: ``batch`` fresh requests prefilled; W untimed and K timed steps through
        ``LLMEngine.step()`` (end to end: host tokens in and out); W untimed and K timed steps enqueued
        back to back through the step function (device time, CUDA events).  One engine serves all
        repeats, so its decode graphs are captured once."""
        engine = make_engine(batch, 2 * steps)
        runner, cache = engine.runner, engine.cache
        dev_ms, e2e_ms = [], []
        result: dict = {}
        total = 0.0
        while total < target_s and len(dev_ms) < (1 if once else MAX_REPEATS):
            ids = fill(engine, batch, steps)
            assert len(ids) == batch
            ctx_start = cache.get(ids[0]).num_computed
            # ---- end to end: the engine's own loop, host tokens in and out -------------------------------
            for _ in range(warmup):
                engine.step()
            torch.cuda.synchronize()
            if sampler is not None and not dev_ms:
                sampler.mark()
            l0 = launch_count() + runner.graph_kernel_launches
            up0 = runner.uploaded_bytes
            t0 = time.perf_counter()
            for _ in range(steps):
                outs = engine.step()
                assert len(outs) == batch
            torch.cuda.synchronize()
            e2e_s = time.perf_counter() - t0
            e2e_launches = launch_count() + runner.graph_kernel_launches - l0
            h2d = (runner.uploaded_bytes - up0) / steps  # (steps that only go on from device state upload nothing)
            # ---- device-timed: the same kind of steps enqueued back to back ---------------------------------
            tokens = [[rng.randrange(vocab)] for _ in range(batch)]
            ctx_now = cache.get(ids[0]).num_computed
            step_fn = engine.decode_step_device
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for _ in range(warmup):
                step_fn(ids, tokens)
            torch.cuda.synchronize()
            l0 = launch_count() + runner.graph_kernel_launches
            start.record()
            for _ in range(steps):
                step_fn(ids, tokens)
            end.record()
            torch.cuda.synchronize()
            ms = start.elapsed_time(end)
            launches = launch_count() + runner.graph_kernel_launches - l0
            runner.check_status()
            dev_ms.append(ms / steps)
            e2e_ms.append(e2e_s * 1e3 / steps)
            total += ms / 1e3 + e2e_s
            if args.timeline and not result:
                print_timeline(step_fn, ids, tokens)
            ctx_mid = ctx_now + warmup + steps // 2
            result = {"launches": launches, "e2e_launches": e2e_launches, "h2d_bytes": h2d, "d2h_bytes": batch * 4 + 16,
                      "ctx_start": ctx_start, "ctx_mid": ctx_mid,
                      "bytes": model.weight_bytes() + batch * ctx_mid * cache.bytes_per_token()}
            drain(engine)
        ms, e2e = statistics.median(dev_ms), statistics.median(e2e_ms)
        result.update(batch=batch, steps=steps, ms_per_step=ms, tok_s=batch / (ms / 1e3), e2e_ms_per_step=e2e,
                      e2e_tok_s=batch / (e2e / 1e3), repeats=spread(dev_ms), e2e_repeats=spread(e2e_ms))
        del engine
        torch.cuda.empty_cache()
        return result

    def time_span(batch: int) -> dict:
        """Every decode step of the benchmark's span, contexts 1,024 to 1,280, device-timed in one piece."""
        engine = make_engine(batch, GENERATED)
        ids = fill(engine, batch, GENERATED)
        tokens = [[rng.randrange(vocab)] for _ in range(batch)]
        step_fn = engine.decode_step_device
        first = engine.cache.get(ids[0]).num_computed
        for _ in range(3):
            step_fn(ids, tokens)
        steps = PROMPT_LEN + GENERATED - engine.cache.get(ids[0]).num_computed
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            step_fn(ids, tokens)
        end.record()
        torch.cuda.synchronize()
        engine.runner.check_status()
        ms = start.elapsed_time(end) / steps
        last_bytes = model.weight_bytes() + batch * (PROMPT_LEN + GENERATED) * engine.cache.bytes_per_token()
        mean_bytes = model.weight_bytes() + batch * (first + 3 + steps / 2) * engine.cache.bytes_per_token()
        drain(engine)
        del engine
        torch.cuda.empty_cache()
        return {"tok_s": batch / (ms / 1e3), "ms_per_step": ms, "steps": steps,
                "hbm_frac": mean_bytes / (ms / 1e3) / 1e9 / peak["hbm_gbs"], "bytes_at_1280": last_bytes}

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

    def time_prefill(reps: int = 5, tokens: int = PREFILL_LEN) -> dict:
        """One prompt of ``tokens`` tokens through the step function, wall clock of the device (events around
        the call: a short prompt's step is a captured graph, and the host's share of a step counts)."""
        engine = make_engine(1, 1)
        runner, cache = engine.runner, engine.cache
        times = []
        for rep in range(reps + 2):
            rid = f"p{rep}"
            cache.open(rid)
            toks = [rng.randrange(vocab) for _ in range(tokens)]
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            logits = runner.step([StepEntry(rid, toks, [tokens - 1])])
            end.record()
            torch.cuda.synchronize()
            assert logits.shape == (1, vocab)
            if rep >= 2:
                times.append(start.elapsed_time(end))
            cache.close(rid)
        runner.check_status()
        ms = statistics.median(times)
        flops = prefill_flops(raw, tokens)
        del engine
        torch.cuda.empty_cache()
        return {"value": tokens / (ms / 1e3), "tokens": tokens, "ms": ms,
                "frac": flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12), "tflops": flops / (ms / 1e3) / 1e12,
                "repeats": spread(times)}

    def time_mixed(reps: int = 7, decodes: int = 32, ctx: int = 2048, portions: int = 2, portion_len: int = 512) -> dict:
        """One step of ``decodes`` single tokens at context ``ctx`` beside ``portions`` prompt portions of
        ``portion_len`` tokens (the workload of the benchmark description's fourth configuration, at this
        model's sizes): device time of the step function, the portions being new prompts every time."""
        engine = make_engine(decodes + portions, reps + 4, num_blocks=(decodes * (ctx + 64) + portions * portion_len) // PAGE + 64,
                             max_num_seqs=decodes + portions)
        runner, cache = engine.runner, engine.cache
        ids = fill(engine, decodes, reps + 4, prompt_len=ctx - 4)
        engine._launched = None
        times = []
        for rep in range(reps + 2):
            entries = [StepEntry(rid, [rng.randrange(vocab)], [0]) for rid in ids]
            fresh = [f"q{rep}_{j}" for j in range(portions)]
            for rid in fresh:
                cache.open(rid)
                entries.append(StepEntry(rid, [rng.randrange(vocab) for _ in range(portion_len)], [portion_len - 1]))
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            logits = runner.step(entries)
            end.record()
            torch.cuda.synchronize()
            assert logits.shape[0] == decodes + portions
            if rep >= 2:
                times.append(start.elapsed_time(end))
            for rid in fresh:
                cache.close(rid)
        runner.check_status()
        ms = statistics.median(times)
        tokens = decodes + portions * portion_len
        h, nh, nkv, hd = raw["hidden_size"], raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"]
        per_layer = h * (nh + 2 * nkv) * hd + nh * hd * h + 3 * h * raw["intermediate_size"]
        flops = (2 * per_layer * len(model.spec.layers) * tokens + 2 * h * vocab * (decodes + portions)
                 + len(model.spec.layers) * 4 * nh * hd * (decodes * ctx + portions * portion_len * (portion_len + 1) / 2))
        step_bytes = model.weight_bytes() + decodes * ctx * cache.bytes_per_token()
        drain(engine)
        del engine
        torch.cuda.empty_cache()
        return {"ms": ms, "tokens": tokens, "tok_s": tokens / (ms / 1e3), "decodes": decodes, "decode_ctx": ctx,
                "portions": portions, "portion_len": portion_len,
                "flops_frac": flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12),
                "hbm_frac": step_bytes / (ms / 1e3) / 1e9 / peak["hbm_gbs"], "repeats": spread(times)}

    def time_shared_prefix(requests: int = 64, prefix_len: int = 1536, suffix_len: int = 256, new_tokens: int = 128) -> dict:
        """``requests`` prompts that share their first ``prefix_len`` tokens, each with its own suffix, through
        ``LLMEngine.generate`` with the prefix cache on (the pattern of the benchmark description's fifth
        configuration, at this model's sizes): how long admission takes, how many prompt tokens came from
        the cache, and the decode rate once all requests run."""
        tokens_per_seq = prefix_len + suffix_len + new_tokens + PAGE
        engine = make_engine(requests, new_tokens, enable_prefix_cache=True, max_num_seqs=requests,
                             num_blocks=requests * ((tokens_per_seq + PAGE - 1) // PAGE) + 64)
        params = SamplingParams(max_tokens=new_tokens, ignore_eos=True)
        cached0 = prompt0 = 0
        for timed_pass in (False, True):
            # (the first pass, with a prefix of its own, is not timed: the steps' graphs are captured in it)
            if timed_pass:
                stats = engine.stats()
                cached0, prompt0 = stats["total_cached_tokens"], stats["total_prompt_tokens"]
            shared = [rng.randrange(vocab) for _ in range(prefix_len)]
            for i in range(requests):
                engine.add_request(f"r{int(timed_pass)}_{i}", prompt_token_ids=shared + [rng.randrange(vocab) for _ in range(suffix_len)],
                                   sampling_params=params)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            admission_steps = 0
            while engine.scheduler.waiting or any(s.num_uncomputed_tokens() > 1 for s in engine.scheduler.running):
                engine.step()
                admission_steps += 1
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            decode_steps = 0
            while engine.has_unfinished_requests():
                engine.step()
                decode_steps += 1
            torch.cuda.synchronize()
            t2 = time.perf_counter()
        stats = engine.stats()
        del engine
        torch.cuda.empty_cache()
        return {"requests": requests, "prefix_len": prefix_len, "suffix_len": suffix_len, "new_tokens": new_tokens,
                "admission_s": t1 - t0, "admission_steps": admission_steps,
                "admission_steps_per_s": admission_steps / (t1 - t0),
                "prompt_tok_s": requests * (prefix_len + suffix_len) / (t1 - t0),
                "cached_tokens": stats["total_cached_tokens"] - cached0, "prompt_tokens": stats["total_prompt_tokens"] - prompt0,
                "decode_tok_s": requests * decode_steps / (t2 - t1), "decode_steps": decode_steps, "total_s": t2 - t0}

    def time_long_prompt(total: int = 32768, portion: int = PREFILL_LEN, reps: int = 2) -> dict:
        """One prompt of ``total`` tokens through the step function in portions of ``portion`` tokens, as the
        scheduler cuts it under its token budget: device time of the whole prompt and of its last portion."""
        engine = make_engine(1, 1, num_blocks=(total + PAGE) // PAGE + 8, max_model_len=total + PAGE)
        runner, cache = engine.runner, engine.cache
        whole, last = [], []
        for rep in range(reps + 1):
            rid = f"long{rep}"
            cache.open(rid)
            per_step = []
            for first in range(0, total, portion):
                toks = [rng.randrange(vocab) for _ in range(min(portion, total - first))]
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                start.record()
                runner.step([StepEntry(rid, toks, [len(toks) - 1])])
                end.record()
                torch.cuda.synchronize()
                per_step.append(start.elapsed_time(end))
            cache.close(rid)
            if rep >= 1:
                whole.append(sum(per_step))
                last.append(per_step[-1])
        runner.check_status()
        ms = statistics.median(whole)
        flops = prefill_flops(raw, total) + 2 * raw["hidden_size"] * vocab * (-(-total // portion) - 1)
        del engine
        torch.cuda.empty_cache()
        return {"tokens": total, "portion": portion, "ms": ms, "tok_s": total / (ms / 1e3), "last_portion_ms": statistics.median(last),
                "flops_frac": flops / (ms / 1e3) / (peak["bf16_tflops"] * 1e12)}

    if args.only == "long-prompt":
        print(json.dumps({"impl": "ours", "long_prompt": time_long_prompt(total=args.prompt_len or 32768)}))
        return 0
    if args.only == "prefill":
        print(json.dumps({"impl": "ours", "prefill": time_prefill(reps=1 if args.prompt_len is None else 5,
                                                                   tokens=args.prompt_len or PREFILL_LEN)}))
        return 0
    if args.only == "mixed":
        print(json.dumps({"impl": "ours", "mixed": time_mixed(reps=1)}))
        return 0
    if args.only == "shared-prefix":
        print(json.dumps({"impl": "ours", "shared_prefix": time_shared_prefix()}))
        return 0
    with ClockSampler() as clocks:
        clocks.wait_for_first_line()
        main_run = time_decode(args.batch, args.steps, args.warmup, clocks)
    if args.only == "decode":
        print(json.dumps({"impl": "ours", "batch": args.batch, "context": main_run["ctx_mid"], "ms_per_step": main_run["ms_per_step"],
                          "tok_s": main_run["tok_s"], "e2e_tok_s": main_run["e2e_tok_s"], "launches": main_run["launches"],
                          "hbm_frac": main_run["bytes"] / (main_run["ms_per_step"] / 1e3) / 1e9 / peak["hbm_gbs"]}))
        return 0
    hbm_frac = main_run["bytes"] / (main_run["ms_per_step"] / 1e3) / 1e9 / peak["hbm_gbs"]
    out = {
        "metric": "decode tokens/s (Qwen2.5-1.5B shape, random weights)",
        "value": main_run["tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": main_run["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": config_record(raw, full_layers, args.batch, main_run["ctx_mid"], peak_kind),
        "clocks": clocks.summary(), "repeats": main_run["repeats"],
        "e2e": {"value": main_run["e2e_tok_s"], "unit": "tok/s", "ms_per_step": main_run["e2e_ms_per_step"],
                "h2d_bytes_per_step": main_run["h2d_bytes"], "d2h_bytes_per_step": main_run["d2h_bytes"],
                "repeats": main_run["e2e_repeats"]},
        "gpu_launches": main_run["launches"],
        "roofline": {"bound": "hbm", "achieved": hbm_frac * peak["hbm_gbs"], "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": hbm_frac, "bytes_per_step": main_run["bytes"], "of": peak_kind},
    }
    if not args.skip_points:
        out["prefill"] = time_prefill()
        points = {}
        for batch in (1, 64):
            r = time_decode(batch, max(16, args.steps // 2), args.warmup, target_s=0.5)
            points[f"decode_b{batch}"] = r["tok_s"]
            points[f"decode_b{batch}_e2e"] = r["e2e_tok_s"]
            points[f"decode_b{batch}_hbm_frac"] = r["bytes"] / (r["ms_per_step"] / 1e3) / 1e9 / peak["hbm_gbs"]
        span = time_span(args.batch)
        points["decode_span_1024_1280"] = span["tok_s"]
        points["decode_span_1024_1280_hbm_frac"] = span["hbm_frac"]
        for tokens in (32, 128, 512):
            points[f"prefill_{tokens}_ms"] = time_prefill(tokens=tokens)["ms"]
        small = time_mixed(decodes=7, ctx=1024, portions=1, portion_len=256)
        points["mixed_7x1024_1x256_ms"] = small["ms"]
        long_prompt = time_long_prompt()
        points["long_prompt_32768_tok_s"] = long_prompt["tok_s"]
        points["long_prompt_32768_flops_frac"] = long_prompt["flops_frac"]
        points["prefill_2048_behind_30720_ms"] = long_prompt["last_portion_ms"]
        mixed = time_mixed()
        points["mixed_32x2048_2x512_tok_s"] = mixed["tok_s"]
        points["mixed_32x2048_2x512_ms"] = mixed["ms"]
        points["mixed_32x2048_2x512_flops_frac"] = mixed["flops_frac"]
        points["mixed_32x2048_2x512_hbm_frac"] = mixed["hbm_frac"]
        shared = time_shared_prefix()
        points["shared_prefix_64x1536_decode_tok_s"] = shared["decode_tok_s"]
        points["shared_prefix_64x1536_admission_s"] = shared["admission_s"]
        points["shared_prefix_64x1536_admission_steps_per_s"] = shared["admission_steps_per_s"]
        points["shared_prefix_64x1536_cached_frac"] = shared["cached_tokens"] / max(1, shared["prompt_tokens"])
        out["points"] = points
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
