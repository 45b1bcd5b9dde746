"""Measurements on random-weight models of given shapes: what `bench.py` prints and what
`python -m reinfer_b200 bench` shows.  A shape is a config.json: one of the files under
`reinfer_b200/shapes/` (qwen3-8b, qwen3-4b, qwen3-32b: the three sizes the measurements are
quoted on) or any path.  The model is built through the registry like every other, with
weights drawn on the device by the seeded generator, and driven through the public entry
points: `Engine.step` for the prefill, `LLM.step` for decoding and for the mixed run.

The reference measures through `run --perf` (bin/reinfer/src/main.rs:700-727) and an HTTP
load generator (bench/gate-fixture.md:24-28, bench/notes.md:1534: concurrent requests);
here seeded uniform-random token ids of the stated lengths stand in for any data set.

  prefill(T)            one request of T tokens in one step; tokens/s and the fraction of the
                        tensor-core peak (flops of the products and of causal attention / time)
  decode(B, ...)        B requests at a given context decode together; per step: the device's
                        time (the captured step - every layer, the head, the sampler - replayed
                        back to back) and the time through `LLM.step` (scheduler, tables from
                        pinned memory, graph, sampler, ids back to pinned memory)
  mixed(n, lo, hi, ...) n requests with prompt lengths uniform in [lo, hi] arrive at once; prompts
                        are cut under the token budget and run beside the others' decode tokens
  segments(...)         one step launched eagerly with an event behind every launch: time, achieved
                        TFLOP/s and GB/s by kernel family
"""
from __future__ import annotations

import json
import os
import time
from typing import Dict, List, Optional

SHAPES_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "shapes")


def shape_path(name: str) -> str:
    """A shape's config.json: a path, or the name of a file under reinfer_b200/shapes (with or without the family's
    prefix: '8b' = 'qwen3-8b')."""
    if os.path.isfile(name):
        return name
    if os.path.isfile(os.path.join(name, "config.json")):
        return os.path.join(name, "config.json")
    known = sorted(f[:-5] for f in os.listdir(SHAPES_DIR) if f.endswith(".json"))
    for cand in known:
        if name.lower() == cand or cand.endswith("-" + name.lower()):
            return os.path.join(SHAPES_DIR, cand + ".json")
    raise FileNotFoundError(f"shape {name!r}: not a config.json and not one of {known}")


def load_shape(name: str, layers: Optional[int] = None):
    """(raw config, typed config, layers of the full model).  `layers` builds fewer layers of the same sizes."""
    from .config.registry import resolve_architecture
    with open(shape_path(name)) as f:
        raw = json.load(f)
    full = int(raw.get("num_hidden_layers", 0))
    if layers:
        raw["num_hidden_layers"] = int(layers)
    arch = resolve_architecture(raw)
    return raw, arch.config_cls.from_dict(raw), full


def peaks(root: Optional[str] = None):
    """(copy GB/s, bf16 TFLOP/s burst, sustained, 'measured'|'fallback') from MEASURED_PEAKS.json beside the package."""
    root = root or os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, 1590.0, 1400.0, "fallback"


class Bench:
    """One engine of one shape, and the runs on it."""

    def __init__(self, shape: str, layers: Optional[int] = None, page_size: int = 16, dtype: str = "bfloat16",
                 pool_tokens: int = 0, max_num_seqs: int = 65, seed: int = 0, memory_fraction: float = 0.9):
        import torch
        from .engine import Engine
        self.torch = torch
        self.raw, self.cfg, self.full_layers = load_shape(shape, layers)
        self.layers = int(self.raw["num_hidden_layers"])
        t0 = time.time()
        kw = dict(max_tokens=pool_tokens) if pool_tokens else dict(memory_fraction=memory_fraction)
        self.engine = Engine.from_config(self.cfg, seed=seed, dtype=dtype, page_size=page_size,
                                         max_num_seqs=max_num_seqs, **kw)
        torch.cuda.synchronize()
        self.load_s = time.time() - t0
        self.page_size = page_size
        self.vocab = self.engine.vocab_size
        self.gen = torch.Generator().manual_seed(seed)
        self._account()

    # ---- what a step has to move and to compute ------------------------------------------------------
    def _account(self) -> None:
        """Bytes of the weights that a step reads once (every tensor but a gathered embedding table), bytes of cache
        per token, and the multiply-adds per token of the products."""
        model = self.engine.model
        spec = model.spec
        isz = 2 if self.engine.dtype == self.torch.bfloat16 else 4
        tied = bool(getattr(model.lm_head, "tied", False))
        total = mat = 0
        for name, ps in model.param_specs().items():
            n = 1
            for s in ps.shape:
                n *= s
            if name == spec.embedding.prefix + "weight":
                if tied:
                    total += n                              # read as the output matrix
                continue
            if name.startswith(spec.lm_head.prefix) and ps.optional and tied:
                continue
            total += n
            if len(ps.shape) == 2 and not name.startswith(spec.lm_head.prefix):
                mat += n
        self.weight_bytes = total * isz
        self.matmul_params = mat                            # without the output matrix (it runs on wanted rows only)
        self.head_params = spec.vocab_size * spec.hidden_size
        paged, _ = model.cache_layout()
        self.kv_bytes_per_token = sum(2 * s.kv_heads * s.head_dim * isz for s in paged.values())
        self.attn_dims = [(l.mixer.QH, l.mixer.d) for i, _ in model.run for l in [model.layers[i]]
                          if l.mixer is not None and hasattr(l.mixer, "QH")]

    def prefill_flops(self, T: int, rows: int = 1) -> float:
        attn = sum(4.0 * qh * d * T * (T + 1) / 2 for qh, d in self.attn_dims)     # QK^T and PV over the causal half
        return 2.0 * T * self.matmul_params + attn + 2.0 * rows * self.head_params

    def tokens(self, n: int) -> List[int]:
        return self.torch.randint(0, self.vocab, (n,), generator=self.gen).tolist()

    def _ev(self):
        return self.torch.cuda.Event(enable_timing=True)

    # ---- prefill -------------------------------------------------------------------------------------
    def prefill(self, T: int = 2048, repeats: int = 3) -> Dict:
        from .engine import StepEntry
        torch, ms = self.torch, []
        for it in range(repeats):
            toks = self.tokens(T)
            e0, e1 = self._ev(), self._ev()
            torch.cuda.synchronize()
            e0.record()
            self.engine.step([StepEntry("prefill", toks, [T - 1])])
            e1.record()
            torch.cuda.synchronize()
            ms.append(e0.elapsed_time(e1))
            self.engine.finish("prefill")
        best = min(ms[1:]) if len(ms) > 1 else ms[0]
        return {"tokens": T, "ms": best, "value": T / best * 1e3, "flops": self.prefill_flops(T)}

    # ---- decode --------------------------------------------------------------------------------------
    def decode(self, B: int, steps: int, warmup: int, context: int) -> Dict:
        """Fill B requests so that they are at about `context` tokens when the timed steps end; time `steps` steps
        through `LLM.step` by the wall clock, then the same step's graph alone by CUDA events."""
        from .engine.llm import LLM
        from .sampling import SamplingParams
        torch, engine = self.torch, self.engine
        # the request admitted first decodes while the others still run their prompts (a prompt takes context / 2,048
        # steps): leave that many tokens of room, so that no request passes `context` (and no block table outgrows the
        # captured step's width) before the timed steps end
        start_len = max(context - steps - warmup - B * (-(-context // 2048) + 1) - 2, 1)
        llm = LLM(engine=engine, max_batch_tokens=2048, seed=0)
        sp = SamplingParams(temperature=0.0, max_tokens=1 << 20, ignore_eos=True)
        for _ in range(B):
            llm.add_request(self.tokens(start_len), sp)
        while any(r.in_prefill for r in llm.scheduler.running) or llm.scheduler.waiting:
            llm.step()
        for _ in range(warmup):
            llm.step()
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        for _ in range(steps):
            llm.step()
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - w0) / steps * 1e3
        if len(llm.scheduler.running) != B or llm.scheduler.waiting:
            raise RuntimeError("decode run: a request left the batch during the timed steps")
        kv_tokens = sum(engine.cache.length(r.request_id) for r in llm.scheduler.running)
        bucket = B if B <= 8 else -(-B // 8) * 8
        graph = max((g for key, g in engine._graphs.items() if key[0] == bucket), key=lambda g: g.meta.numel())
        for _ in range(3):
            graph.graph.replay()
        torch.cuda.synchronize()
        e0, e1 = self._ev(), self._ev()
        e0.record()
        for _ in range(steps):
            graph.graph.replay()
        e1.record()
        torch.cuda.synchronize()
        dev_ms = e0.elapsed_time(e1) / steps
        out = {"batch": B, "context": context, "ms_device": dev_ms, "ms_e2e": wall_ms, "launches_per_step": graph.n_launches,
               "kv_tokens": kv_tokens, "bytes": self.weight_bytes + kv_tokens * self.kv_bytes_per_token,
               "h2d_bytes_per_step": int(graph.meta.numel()) * 4, "d2h_bytes_per_step": B * 4,
               "steps_launched_ahead": llm.steps_launched_ahead}
        for r in list(llm.scheduler.running):
            llm.abort(r.request_id)
        while llm.has_work():
            llm.step()                                    # a step launched ahead is read and dropped
        return out

    # ---- many requests at once ----------------------------------------------------------------------------
    def mixed(self, n_requests: int = 32, lo: int = 128, hi: int = 4096, budget: int = 2048, new_tokens: int = 128,
              seed: int = 0, passes: int = 2) -> Dict:
        """`n_requests` arrive together with prompt lengths uniform in [lo, hi]; every one generates `new_tokens`.
        The same requests run `passes` times through one entry point and the last pass is the one reported: the
        passes before it pay for what a serving process pays once (first launches, the captures of the decode
        steps' graphs, which belong to the entry point's sampler and go with it)."""
        from .engine.llm import LLM
        from .sampling import SamplingParams
        torch = self.torch
        g = torch.Generator().manual_seed(seed)
        lengths = torch.randint(lo, hi + 1, (n_requests,), generator=g).tolist()
        prompts = [self.tokens(n) for n in lengths]
        llm = LLM(engine=self.engine, max_batch_tokens=budget, seed=seed)
        sp = SamplingParams(temperature=0.0, max_tokens=new_tokens, ignore_eos=True)
        for _ in range(max(1, passes)):
            ids = [llm.add_request(p, sp) for p in prompts]
            ahead0, pre0 = llm.steps_launched_ahead, llm.scheduler.stats["preemptions"]
            first: Dict = {}
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            steps = 0
            while llm.has_work():
                llm.step()
                steps += 1
                now = time.perf_counter() - t0
                for rid in ids:
                    if rid not in first and llm.requests[rid].output:
                        first[rid] = now
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            gen = sum(len(llm.requests.pop(rid).output) for rid in ids)
        ttft = sorted(first.values())
        return {"requests": n_requests, "prompt_tokens": sum(lengths), "generated_tokens": gen, "seconds": dt, "steps": steps,
                "tokens_per_s": (sum(lengths) + gen) / dt, "generated_per_s": gen / dt, "budget": budget,
                "preemptions": llm.scheduler.stats["preemptions"] - pre0, "ttft_p50_s": ttft[len(ttft) // 2] if ttft else None,
                "ttft_max_s": ttft[-1] if ttft else None, "steps_launched_ahead": llm.steps_launched_ahead - ahead0,
                "passes": max(1, passes)}

    # ---- where a step's time goes ----------------------------------------------------------------------------
    def segments(self, kind: str, B: int = 8, context: int = 4096, T: int = 2048) -> Dict:
        """One step of the kind ('decode': B requests at `context`; 'prefill': T tokens), launched eagerly with an
        event behind every launch (ops.SegmentProfiler).  -> name -> {n, us, tflops, gbs}."""
        from . import ops
        from .engine import StepEntry
        torch, engine = self.torch, self.engine
        graphs, engine.cuda_graphs = engine.cuda_graphs, False
        prof = ops.SegmentProfiler()
        try:
            if kind == "decode":
                for b in range(B):
                    toks = self.tokens(context - 2)
                    for i in range(0, len(toks), 2048):
                        engine.step([StepEntry(("seg", b), toks[i:i + 2048], [])])
                entries = [StepEntry(("seg", b), [5 + b], [0]) for b in range(B)]
                engine.step(entries)                                    # warm
                entries = [StepEntry(("seg", b), [7 + b], [0]) for b in range(B)]
            else:
                engine.step([StepEntry(("seg", "w"), self.tokens(T), [T - 1])])
                engine.finish(("seg", "w"))
                entries = [StepEntry(("seg", 0), self.tokens(T), [T - 1])]
            torch.cuda.synchronize()
            # the host needs a few milliseconds to queue a step's launches and events: the device sleeps meanwhile, so
            # that no launch waits for the host and a launch's span is the kernel's own time
            torch.cuda._sleep(60_000_000 if kind == "decode" else 20_000_000)
            old = ops.set_profiler(prof)
            prof.begin()
            try:
                engine.step(entries)
            finally:
                ops.set_profiler(old)
            out = prof.summary()
        finally:
            engine.cuda_graphs = graphs
            for rid in list(engine.cache.live()):
                if isinstance(rid, tuple) and rid and rid[0] == "seg":
                    engine.finish(rid)
        return out


def segment_table(seg: Dict, hbm_gbs: float, tflops: float) -> List[str]:
    """Lines of a table: family, launches, microseconds, share, achieved rate and its fraction of the peak."""
    total = sum(d["us"] for d in seg.values()) or 1.0
    lines = [f"{'segment':28s} {'n':>4s} {'us':>9s} {'share':>6s} {'TFLOP/s':>8s} {'GB/s':>8s} {'of peak':>8s}"]
    for name, d in sorted(seg.items(), key=lambda kv: -kv[1]["us"]):
        frac = max(d["tflops"] / tflops, d["gbs"] / hbm_gbs)
        lines.append(f"{name:28s} {d['n']:4d} {d['us']:9.1f} {100 * d['us'] / total:5.1f}% {d['tflops']:8.1f} {d['gbs']:8.0f} {100 * frac:7.1f}%")
    lines.append(f"{'total':28s} {sum(d['n'] for d in seg.values()):4d} {total:9.1f}")
    return lines


def compact_segments(seg: Dict, top: int = 6) -> Dict:
    """The `top` segments by time as {name: [us, TFLOP/s, GB/s]} for a one-line record."""
    keep = sorted(seg.items(), key=lambda kv: -kv[1]["us"])[:top]
    return {k: [round(d["us"], 1), round(d["tflops"], 1), round(d["gbs"])] for k, d in keep}


# ------------------------------------------------------------------ two designs side by side
def silutar_shape(width: int, heads: int, ff: int, layers: int, vocab: int = 32768, chunk: int = 1024, head_dim: int = 128,
                  kv_heads: int = 0, positions: int = 8192) -> Dict:
    """A Silutar config.json at layer sizes that resemble a real model's: `layers` layers that cycle through the
    three mixers (parallel, channel_delta, gla), heads of `head_dim`, low-rank maps of width / 16."""
    kv = kv_heads or max(1, heads // 4)
    rank = max(16, width // 16)
    mixers = [
        {"type": "parallel", "mixer": {"left": {"heads": heads, "kv_heads": kv, "dim": head_dim, "vdim": head_dim, "conv": 4,
                                                "mask": {"size": chunk}, "scale": head_dim ** -0.5},
                                       "right": {"heads": heads, "dim": head_dim // 2, "decay_rank": rank},
                                       "left_scale": 0.5, "right_scale": 0.5}},
        {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": head_dim, "vdim": head_dim, "conv": 4,
                                            "decay_rank": rank, "gate_rank": rank}},
        {"type": "gla", "mixer": {"heads": heads, "dim": head_dim // 2, "vdim": head_dim, "tau": 16.0, "decay_rank": rank}},
    ]
    return {"architecture": "Silutar", "vocab": vocab, "width": width, "max_positions": positions, "norm": {"eps": 1e-6},
            "logit_softcap": 30.0,
            "layers": [dict(mixers[i % 3], mlp={"kind": "dense", "ff": ff}) for i in range(layers)]}


def damadra_shape(width: int, heads: int, ff: int, layers: int, vocab: int = 32768, window: int = 1024, head_dim: int = 128,
                  kv_heads: int = 0, experts: int = 8, identity: int = 2, top: int = 3) -> Dict:
    """A Damadra config.json at layer sizes that resemble a real model's: `layers` layers that cycle through a causal
    layer, a windowed layer and a causal layer that reads the keys and values of the causal layer two before it; dense
    feed-forwards of `ff` alternate with mixtures of `experts` experts of ff / 4 (plus identity experts); heads of
    `head_dim`, bias tables of 32 rows up to a distance of 512."""
    kv = kv_heads or max(1, heads // 4)
    base = {"heads": heads, "kv_heads": kv, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5, "bias_max": 512,
            "bias_rows": 32}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": max(8, ff // 4)}, "router": {"experts": experts, "identity": identity, "top": top}}
    out = []
    for i in range(layers):
        if i % 3 == 1:
            layer = {"type": "attention", "mixer": dict(base, mask={"size": window})}
        else:
            layer = {"type": "attention_2", "mixer": dict(base, q_temp={"coef": 0.25, "every": 128})}
            if i % 3 == 2:
                layer["mixer"]["kv_from"] = i - 2
        out.append(dict(layer, mlp=moe if i % 2 else dense))
    return {"architecture": "Damadra", "vocab": vocab, "width": width, "embedding": {"scale": float(width) ** 0.5},
            "norm": {"eps": 1e-6}, "residual_mult": 0.4, "layers": out}


def molitar_shape(width: int, heads: int, ff: int, layers: int, vocab: int = 32768, head_dim: int = 128, kv_heads: int = 0,
                  kv_rank: int = 192, rot_dim: int = 64) -> Dict:
    """A Molitar config.json at layer sizes that resemble a real model's: `layers` layers of which every third (the
    second, the fifth, ...) is a gated attention layer (heads of `head_dim` over heads / 4 key/value heads, half of each
    head rotated, a soft cap of 30, a sink, value mixing and an output gate) and the others latent attention layers
    (heads of `head_dim` + `rot_dim`, values of `head_dim`, a query bottleneck of 3/4 of the width and a latent of
    `kv_rank`: a token's cached row is kv_rank + rot_dim numbers, stretched rotation), all with dense feed-forwards."""
    kv = kv_heads or max(1, heads // 4)
    latent = {"heads": heads, "dim": head_dim, "rot_dim": rot_dim, "vdim": head_dim, "q_rank": 3 * width // 4, "kv_rank": kv_rank,
              "scale": (head_dim + rot_dim) ** -0.5,
              "rot": {"base": 10000.0, "dims": rot_dim, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    gated = {"heads": heads, "kv_heads": kv, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5, "softcap": 30.0, "v_mix": True,
             "rot": {"base": 1e6, "dims": head_dim // 2}}
    out = [{"type": "attention", "mixer": gated, "mlp": {"kind": "dense", "ff": ff}} if i % 3 == 1 else
           {"type": "latent_attention", "mixer": latent, "mlp": {"kind": "dense", "ff": ff}} for i in range(layers)]
    return {"architecture": "Molitar", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "residual_mult": 0.4, "logit_scale": 0.5,
            "layers": out}


def zegorax_shape(width: int, heads: int, ff: int, layers: int, vocab: int = 32768, head_dim: int = 128, kv_heads: int = 0,
                  kv_rank: int = 192, rot_dim: int = 64, window: int = 1024, experts: int = 8, top: int = 2, positions: int = 8192) -> Dict:
    """A Zegorax config.json at layer sizes that resemble a real model's: the layers cycle differential attention (heads / 2
    heads of two maps of head_dim each over an eighth as many key heads, values of head_dim - the query and key projections
    are as large as those of `heads` plain heads - a quarter of each map rotated with stretched frequencies) -> latent
    attention (heads of head_dim + rot_dim, values of head_dim, a query bottleneck of 3/4 of the width, a latent of kv_rank,
    a window) -> the delta rule with a decay per head (heads of head_dim over heads / 4 key heads, four taps); feed-forwards
    alternate between dense (tanh-gelu, biases) and mixtures of `experts` experts of ff / 4 of which `top` are chosen."""
    kv = kv_heads or max(1, heads // 4)
    pairs = max(1, heads // 2)
    attention = {"heads": pairs, "kv_heads": max(1, pairs // 4), "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5, "diff": 0.2,
                 "rot": {"base": 1e6, "dims": head_dim // 4, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 2048}}}
    latent = {"heads": heads, "dim": head_dim, "rot_dim": rot_dim, "vdim": head_dim, "q_rank": 3 * width // 4, "kv_rank": kv_rank,
              "scale": (head_dim + rot_dim) ** -0.5, "mask": {"size": window}, "rot": {"base": 10000.0, "dims": rot_dim}}
    delta = {"heads": heads, "kv_heads": kv, "dim": head_dim, "vdim": head_dim, "conv": 4}
    mixers = (("attention", attention), ("latent_attention", latent), ("delta", delta))
    out = []
    for i in range(layers):
        kind, m = mixers[i % 3]
        mlp = {"kind": "dense", "ff": ff} if i % 2 == 0 else \
            {"kind": "moe", "expert": {"ff": ff // 4}, "router": {"experts": experts, "top": top}}
        out.append({"type": kind, "mixer": m, "mlp": mlp})
    return {"architecture": "Zegorax", "vocab": vocab, "width": width, "max_positions": positions, "norm": {"eps": 1e-5}, "layers": out}


def qwen3_shape(width: int, heads: int, ff: int, layers: int, vocab: int = 32768, head_dim: int = 128, kv_heads: int = 0,
                positions: int = 8192) -> Dict:
    """The closest existing design at the same layer sizes."""
    return {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "head_dim": head_dim, "vocab_size": vocab,
            "rope_theta": 1e6, "rms_norm_eps": 1e-6, "max_position_embeddings": positions, "num_hidden_layers": layers,
            "hidden_size": width, "num_attention_heads": heads, "num_key_value_heads": kv_heads or max(1, heads // 4),
            "intermediate_size": ff, "tie_word_embeddings": True}


def time_design(raw: Dict, prompt: int = 2048, batch: int = 8, context: int = 2048, steps: int = 32, page_size: int = 16,
                seed: int = 0, segments: bool = True) -> Dict:
    """Random weights of the configuration `raw` on the device; prefill of one `prompt`-token request and decode steps
    of `batch` requests at `context` tokens, both timed on the device by CUDA events (decode: replays of the captured
    step); and one eager step of each kind by kernel family."""
    import torch
    from . import ops
    from .config.registry import resolve_architecture
    from .engine import Engine, StepEntry
    cfg = resolve_architecture(raw).config_cls.from_dict(raw)
    pool = batch * (context + 2 * page_size) + 2 * prompt
    engine = Engine.from_config(cfg, seed=seed, dtype="bfloat16", page_size=page_size, max_tokens=pool, max_num_seqs=batch + 2)
    gen = torch.Generator().manual_seed(seed)
    toks = lambda n: torch.randint(0, engine.vocab_size, (n,), generator=gen).tolist()
    ev = lambda: torch.cuda.Event(enable_timing=True)
    out: Dict = {}
    ms = []
    for _ in range(4):
        e0, e1 = ev(), ev()
        t = toks(prompt)
        torch.cuda.synchronize()
        e0.record()
        engine.step([StepEntry("p", t, [prompt - 1])])
        e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
        engine.finish("p")
    out["prefill_ms"] = min(ms[1:])
    out["prefill_tok_s"] = prompt / out["prefill_ms"] * 1e3
    for b in range(batch):
        t = toks(context - steps - 8)
        for i in range(0, len(t), 2048):
            engine.step([StepEntry(("d", b), t[i:i + 2048], [])])
    for _ in range(4):
        engine.step([StepEntry(("d", b), [3 + b], [0]) for b in range(batch)])
    graph = next(iter(engine._graphs.values())) if engine._graphs else None
    torch.cuda.synchronize()
    e0, e1 = ev(), ev()
    e0.record()
    for _ in range(steps):
        if graph is not None:
            graph.graph.replay()        # the same tokens at the same places again: the step's work is what is timed
        else:
            engine.step([StepEntry(("d", b), [3 + b], [0]) for b in range(batch)])
    e1.record()
    torch.cuda.synchronize()
    out["decode_ms"] = e0.elapsed_time(e1) / steps
    out["decode_tok_s"] = batch / out["decode_ms"] * 1e3
    out["decode_launches"] = graph.n_launches if graph is not None else None
    out["captured"] = graph is not None
    if segments:
        was, engine.cuda_graphs = engine.cuda_graphs, False
        try:
            for kind, entries in (("decode", [StepEntry(("d", b), [9 + b], [0]) for b in range(batch)]),
                                  ("prefill", [StepEntry("s", toks(prompt), [prompt - 1])])):
                if kind == "prefill":
                    # once unmeasured: the decode steps before split the allocator's large blocks, and a prompt's first
                    # step after them waits for new ones - time that the events would put on whatever kernel comes next
                    engine.step([StepEntry("w", toks(prompt), [prompt - 1])])
                    engine.finish("w")
                prof = ops.SegmentProfiler()
                torch.cuda.synchronize()
                torch.cuda._sleep(40_000_000)
                old = ops.set_profiler(prof)
                prof.begin()
                try:
                    engine.step(entries)
                finally:
                    ops.set_profiler(old)
                out[kind + "_segments"] = prof.summary()
        finally:
            engine.cuda_graphs = was
    status = ops.status_word()
    if status:
        raise RuntimeError(f"kernel status word 0x{status:x}")
    del engine
    torch.cuda.empty_cache()
    return out
