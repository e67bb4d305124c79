"""Command-line entry: ``python -m sllm_b200.serving.main <recipe> --mode plan|run``.

Option names and meanings follow the reference's entry (serving/main.py:311-339:
``recipe``, ``--tp/--nodes``, ``--mode``, ``--model-dir``, ``--host``, ``--port``,
``--chat``, ``--max-new``, ``--log-level``, ``--cpu``, ``--placement``, ``--version``)
and its dev command line (serving/cli.py:18-23: ``--temperature``, ``--top-p``,
``--top-k``, ``--seed``).  ``plan`` prints what would run and executes nothing
(serving/main.py:98-153); ``run`` generates once and prints the result
(serving/main.py:250-259).  ``serve`` (the HTTP server), ``--cpu`` and
``--placement um`` (host-memory decode) name things this engine does not have and
are refused with a plain sentence.  Added here: ``--prompt-ids``, ``--dtype``,
``--random-weights SEED``.
"""

from __future__ import annotations

import argparse
import os
import sys
import tempfile

from .. import __version__
from ..config.errors import ConfigError
from ..config.recipe import Recipe, resolve_recipe

RECIPES_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "recipes")
LEVELS = ("TRACE", "DEBUG", "INFO", "WARNING", "ERROR")
_level = "INFO"


def log(level: str, msg: str) -> None:
    """Level-gated lines on stderr (serving/diag.py:86-96)."""
    if LEVELS.index(level) >= LEVELS.index(_level):
        print(f"[sllm {level}] {msg}", file=sys.stderr, flush=True)


def build_plan(recipe: Recipe, model_dir: str | None, settings: dict) -> str:
    lines = [f"sllm plan: {recipe.name}",
             f"  model    : {recipe.model_id} (arch {recipe.arch}, dtype {settings['dtype']})",
             f"  recipe   : {recipe.path}",
             f"  weights  : {model_dir or '(none: give --model-dir or --random-weights)'}"]
    try:
        # what the model asks of the cache comes from the model itself (built without weights), not from
        # keys of one architecture's config.json
        import torch

        from ..cache.manager import CacheManager
        from ..config.registry import architecture_of, load_config
        from ..models.causal_lm import CausalLM
        if model_dir and os.path.isfile(os.path.join(model_dir, "config.json")):
            arch, typed = load_config(model_dir)
        elif recipe.text:
            raw = recipe.config_json()
            arch = architecture_of(raw)
            typed = arch.config_cls.from_dict(raw)
        else:
            arch = typed = None
        if arch is not None:
            plan = arch.plan(typed)
            dt = torch.bfloat16 if settings["dtype"] == "bfloat16" else torch.float32
            model = CausalLM(plan, dtype=dt, device="cpu")
            probe = CacheManager(model.cache_needs(), page_size=settings["block_size"], num_pages=0, max_requests=1)
            per_token = probe.bytes_per_token(2 if dt == torch.bfloat16 else 4)      # runtime/memory_planner.py:12-15
            lines.append(f"  geometry : {arch.name}: {len(plan.layers)} layers in {len(plan.run_list)} runs, hidden "
                         f"{plan.hidden_size}, vocab {plan.vocab_size}, {plan.max_positions} positions")
            budget = (f"{recipe.kv_device_bytes} bytes" if recipe.kv_device_bytes is not None
                      else f"utilisation {recipe.kv_utilization} of the free device memory")
            lines.append(f"  cache    : {per_token} bytes per token, {probe.state_bytes_per_request()} bytes of state per "
                         f"request, pages of {settings['block_size']} tokens, budget {budget}")
            for line in probe.describe():
                lines.append(f"             {line}")
    except (ConfigError, ValueError) as e:
        lines.append(f"  geometry : unreadable ({e})")
    lines.append(f"  schedule : max_num_seqs {settings['max_num_seqs']}, chunk_size {settings['chunk_size']}, "
                 f"max_new {settings['max_new']}")
    lines.append("  nodes    : 1 (mode=plan: nothing executed)")
    return "\n".join(lines)


def main(argv=None) -> int:
    global _level
    ap = argparse.ArgumentParser(prog="sllm", description="sLLM-B200: a one-GPU inference engine")
    ap.add_argument("recipe", nargs="?", help="recipe yaml (path or name under recipes/)")
    ap.add_argument("--tp", "--nodes", dest="nodes", type=int, default=None, metavar="N")
    ap.add_argument("--mode", choices=("plan", "run", "serve"), default="plan")
    ap.add_argument("--model-dir", default=None, help="override recipe paths.local_dir")
    ap.add_argument("--host", default=None)
    ap.add_argument("--port", default=None)
    ap.add_argument("--chat", default=None, help="text of one user turn (byte-level stand-in tokenizer)")
    ap.add_argument("--prompt", default=None, help="raw completion prompt (byte-level stand-in tokenizer)")
    ap.add_argument("--batch", nargs="+", default=None, metavar="PROMPT",
                    help="several prompts served together with continuous batching")
    ap.add_argument("--prompt-ids", default=None, help="comma-separated token ids of the prompt")
    ap.add_argument("--max-new", type=int, default=None)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=None)
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--repetition-penalty", type=float, default=None)
    ap.add_argument("--dtype", choices=("bfloat16", "float32", "bf16", "fp32"), default=None)
    ap.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                    help="write a random model folder from the recipe's geometry and run it")
    ap.add_argument("--log-level", default=None, choices=LEVELS)
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--placement", choices=("device", "um"), default=None)
    ap.add_argument("--version", "-V", action="store_true")
    args = ap.parse_args(argv)
    _level = args.log_level or os.environ.get("SLLM_LOG_LEVEL", "INFO")
    if _level not in LEVELS:
        _level = "INFO"
    if args.version:
        print(f"sllm-b200 {__version__}")
        return 0
    if args.recipe is None:
        ap.error("the following arguments are required: recipe")
    if args.cpu or args.placement == "um":
        raise SystemExit("sllm: this engine has no CPU or host-memory path; it runs on one B200")
    if args.nodes not in (None, 1):
        raise SystemExit(f"sllm: --tp {args.nodes}: this engine runs on one GPU")
    try:
        recipe = resolve_recipe(args.recipe, RECIPES_DIR)
    except ConfigError as e:
        raise SystemExit(f"sllm: {e}") from None
    de = recipe.defaults
    dtype = {"bf16": "bfloat16", "fp32": "float32"}.get(args.dtype, args.dtype) or recipe.dtype
    settings = {
        "dtype": dtype,
        "max_new": args.max_new if args.max_new is not None else int(de.get("max_new", 32)),
        "max_num_seqs": int(de.get("max_num_seqs", 8)), "block_size": int(de.get("block_size", 16)),
        "chunk_size": int(de.get("chunk_size", 512)), "max_model_len": de.get("max_model_len"),
    }
    model_dir = args.model_dir or recipe.local_dir
    if args.mode == "plan":
        print(build_plan(recipe, model_dir, settings))
        return 0
    if args.mode == "serve":
        raise SystemExit("sllm: --mode serve (the HTTP server) is outside this engine; use --mode run or the "
                         "Python entry point sllm_b200.engine.llm.LLM")

    tmp = None
    try:
        if args.random_weights is not None:
            from ..weights import write_random_model
            tmp = tempfile.TemporaryDirectory()
            model_dir = write_random_model(os.path.join(tmp.name, "model"), recipe.config_json(),
                                           args.random_weights, std=0.02, bias_std=0.1)
            log("INFO", f"random weights (seed {args.random_weights}) written to {model_dir}")
        if not model_dir or not os.path.isdir(model_dir):
            raise SystemExit(f"sllm: weights not found: {model_dir or '(no path)'}")     # serving/main.py:239-240
        from ..engine.llm import LLM
        from ..sampling import SamplingParams
        llm = LLM(model_dir, dtype=dtype, block_size=settings["block_size"], max_num_seqs=settings["max_num_seqs"],
                  chunk_size=settings["chunk_size"], max_model_len=settings["max_model_len"],
                  kv_utilization=recipe.kv_utilization, kv_bytes=recipe.kv_device_bytes,
                  progress=lambda d, t: log("INFO", f"load: {d}/{t} tensors"))
        vocab = llm.model.plan.vocab_size
        tok = None
        if args.prompt_ids:
            prompts = [[int(x) for x in args.prompt_ids.replace(" ", "").split(",") if x]]
        else:
            from .tokenizer import ByteTokenizer
            tok = ByteTokenizer(vocab)
            # serving/cli.py:33-54: --batch, else --chat, else --prompt; serving/main.py:256: "hello"
            texts = args.batch or [args.chat if args.chat is not None else (args.prompt if args.prompt is not None else "hello")]
            prompts = [tok.encode(t) for t in texts]
        params = SamplingParams(max_new=settings["max_new"], temperature=args.temperature, top_k=args.top_k,
                                top_p=args.top_p, seed=args.seed, repetition_penalty=args.repetition_penalty)
        import time
        t0 = time.perf_counter()
        results = llm.generate(prompts, params)
        dt = time.perf_counter() - t0
        n_out = sum(len(r.ids) for r in results)
        log("INFO", f"prompt={sum(len(p) for p in prompts)} out={n_out} wall={dt:.3f}s ({n_out / max(dt, 1e-9):.1f} tok/s) "
                    f"finish={','.join(r.finish_reason for r in results)}")           # serving/executor.py:422-427
        for i, res in enumerate(results):
            ids = ",".join(str(t) for t in res.ids)
            if args.batch:                                                              # serving/cli.py:40-41
                print(f"[{args.batch[i]!r}] -> {ids}")
                print(f"[{args.batch[i]!r}] -> {tok.decode(res.ids)!r}")
            else:
                print(ids)
                if tok is not None:
                    print(tok.decode(res.ids))
        return 0
    except ConfigError as e:
        raise SystemExit(f"sllm: {e}") from None
    finally:
        if tmp is not None:
            tmp.cleanup()


if __name__ == "__main__":
    raise SystemExit(main())
