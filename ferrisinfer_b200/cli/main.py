"""Command line in the reference's manner: positional sub-commands with the reference's names.

The reference's CLI (crates/ferrisinfer-cli/src/main.rs:23-167) takes ``<command> [arg] [arg]`` with
the default model folder ``models/Qwen2.5-0.5B-Instruct`` (:19).  The commands that concern the
engine are kept with their names and argument order:

  help                              this message
  plan                              print the parts and run order of the model (the reference prints its step list)
  probe-cuda                        report the CUDA device and whether the kernels load
  inspect-hf [path]                 architecture, sizes, and whether the folder's tensors fit
  profile-hf-load [path]            time config, weights and model set-up
  smoke-hf [ids]                    next-token smoke test: greedy token and its probability
  generate-hf [ids] [tokens]        generate (default 4 new tokens, as the reference)
  profile-hf [ids] [tokens]         time load, prefill and decode (default 1 new token)
  profile-continuous-hf [tokens]    built-in continuous-batching run with staggered arrivals (default 16)

Where the reference takes a text, this CLI takes token ids separated by commas or spaces: text in and
out is the tokenizer's business (the chat, render and tokenize commands are not part of the engine).
Options (all optional, before or after the command): --model DIR, --dtype bfloat16|float32,
--temperature T --top-k K --top-p P --seed S (the reference's sampler fields; default greedy),
--random CONFIG.json --random-seed S (random weights instead of a folder), --page-size, --num-pages.
"""

from __future__ import annotations

import argparse
import json
import sys
import time

DEFAULT_HF_PATH = "models/Qwen2.5-0.5B-Instruct"
COMMANDS = ("help", "plan", "probe-cuda", "inspect-hf", "profile-hf-load", "smoke-hf", "generate-hf", "profile-hf",
            "profile-continuous-hf")


def _parser():
    p = argparse.ArgumentParser(prog="ferrisinfer", add_help=False)
    p.add_argument("command", nargs="?", default="help")
    p.add_argument("args", nargs="*")
    p.add_argument("--model", default=None)
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-k", type=int, default=1)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--random", default=None, help="config.json to build random weights from")
    p.add_argument("--random-seed", type=int, default=0)
    p.add_argument("--page-size", type=int, default=16)
    p.add_argument("--num-pages", type=int, default=None)
    p.add_argument("-h", "--help", action="store_true")
    return p


def _ids(text, default):
    if text is None:
        return list(default)
    return [int(t) for t in text.replace(",", " ").split()]


def _count(text, default):
    return default if text is None else int(text)


def _params(ns, max_new_tokens, stop=None):
    from ..sampling import SamplingParams

    return SamplingParams(temperature=ns.temperature, top_k=ns.top_k, top_p=ns.top_p, seed=ns.seed,
                          max_new_tokens=max_new_tokens, stop_token_id=stop)


def _engine(ns):
    from ..engine.engine import Engine

    if ns.random:
        return Engine(config=ns.random, seed=ns.random_seed, dtype=ns.dtype, page_size=ns.page_size,
                      num_pages=ns.num_pages)
    return Engine(ns.model or DEFAULT_HF_PATH, dtype=ns.dtype, page_size=ns.page_size, num_pages=ns.num_pages)


def _rate(n, seconds):
    """crates/ferrisinfer-cli/src/main.rs:2248-2254."""
    return n / seconds if seconds > 0 else 0.0


def main(argv=None) -> int:
    ns = _parser().parse_args(argv)
    cmd, args = ns.command, ns.args
    out = sys.stdout
    if ns.help or cmd == "help":
        print(__doc__, file=out)
        return 0
    if cmd not in COMMANDS:
        print(f"unknown command: {cmd}", file=sys.stderr)
        print(__doc__, file=out)
        return 1
    try:
        return _run(cmd, args, ns, out)
    except Exception as e:  # the reference prints the error and exits 1 (main.rs:109-112)
        print(f"error: {e}", file=sys.stderr)
        return 1


def _run(cmd, args, ns, out) -> int:
    arg0 = args[0] if args else None
    arg1 = args[1] if len(args) > 1 else None

    if cmd == "probe-cuda":
        import torch

        from ..kernels import build, ops

        ops.require_device()
        props = torch.cuda.get_device_properties(torch.cuda.current_device())
        print(f"device: {props.name}, sm_{props.major}{props.minor}, {props.multi_processor_count} SMs, "
              f"{props.total_memory / 2**30:.1f} GiB", file=out)
        print(f"kernels: {build.library_path(build=False)}", file=out)
        return 0

    if cmd == "inspect-hf":
        from ..weights import inspect_folder

        report = inspect_folder(arg0 or ns.model or DEFAULT_HF_PATH)
        print(json.dumps(report, indent=2), file=out)
        return 0 if report["problems"] is None else 1

    if cmd == "plan":
        from ..config import resolve_config

        arch, cfg = resolve_config(ns.random or ns.model or DEFAULT_HF_PATH)
        plan = arch.plan(cfg)
        print(f"architecture: {plan.architecture}", file=out)
        print(f"embedding: {plan.embedding.kind} {plan.embedding.params}", file=out)
        for i, step in enumerate(plan.run_order):
            lp = plan.layers[step.layer]
            reads = "" if step.cache_of is None else f" (reads the cache of run {step.cache_of})"
            print(f"run {i}: layer {step.layer}{reads}: {lp.mixer_norm.kind} -> {lp.mixer.kind} "
                  f"{ {k: v for k, v in lp.mixer.params.items() if k != 'position'} } -> {lp.feed_forward_norm.kind} "
                  f"-> {lp.feed_forward.kind} {lp.feed_forward.params}", file=out)
        print(f"final norm: {plan.final_norm.kind}; output: {plan.output.kind} {plan.output.params}", file=out)
        return 0

    if cmd == "profile-hf-load":
        import torch

        from ..config import resolve_config
        from ..weights import load_model

        path = arg0 or ns.model or DEFAULT_HF_PATH
        t0 = time.perf_counter()
        resolve_config(path)
        t1 = time.perf_counter()
        load_model(path, ns.dtype, "cuda")
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        from ..weights import SafetensorsFolder

        st = SafetensorsFolder(path)
        stored = sum(e.end - e.begin for e in st.entries.values())
        st.close()
        print(f"config: {(t1 - t0) * 1e3:.1f} ms\nweights + model: {(t2 - t1) * 1e3:.1f} ms "
              f"({stored / 1e9:.2f} GB stored, {stored / 1e9 / max(t2 - t1, 1e-9):.2f} GB/s)\n"
              f"total: {(t2 - t0) * 1e3:.1f} ms", file=out)
        return 0

    import torch

    t0 = time.perf_counter()
    engine = _engine(ns)
    torch.cuda.synchronize()
    load_s = time.perf_counter() - t0
    eos = getattr(engine.config, "eos_token_id", None)

    if cmd == "smoke-hf":
        prompt = _ids(arg0, [0])
        res = engine.generate(prompt, _params(ns, 1))
        tok = res.generated_tokens[0]
        print(f"prompt tokens: {len(prompt)}\nnext token: {tok.token_id}\nprobability: {tok.probability:.6f}", file=out)
        return 0

    if cmd in ("generate-hf", "profile-hf"):
        prompt = _ids(arg0, [0])
        max_new = _count(arg1, 4 if cmd == "generate-hf" else 1)
        t0 = time.perf_counter()
        rid = engine.submit(prompt, _params(ns, max_new, stop=eos))
        first_s = None
        while engine.has_unfinished():
            outs = engine.step()
            if first_s is None and any(o.token is not None or o.finished for o in outs):
                torch.cuda.synchronize()
                first_s = time.perf_counter() - t0
        total_s = time.perf_counter() - t0
        res = engine.output_of(rid)
        ids = res.generated_token_ids()
        print(f"prompt tokens: {len(prompt)}", file=out)
        print(f"generated token ids: {' '.join(str(t) for t in ids)}", file=out)
        print(f"finish reason: {res.finish_reason.value}", file=out)
        if cmd == "profile-hf":
            decode_s = total_s - (first_s or 0.0)
            print(f"load: {load_s * 1e3:.1f} ms", file=out)
            print(f"prefill: {(first_s or 0) * 1e3:.2f} ms ({_rate(len(prompt), first_s or 0):.1f} tok/s)", file=out)
            print(f"decode: {decode_s * 1e3:.2f} ms ({_rate(max(len(ids) - 1, 0), decode_s):.1f} tok/s)", file=out)
        return 0

    if cmd == "profile-continuous-hf":
        # staggered arrivals at steps 0, 2, 4, 6 (crates/ferrisinfer-cli/src/main.rs:1888-1906)
        max_new = _count(arg0, 16)
        vocab = engine.model.vocab_size
        prompts = [[(7 * i + 3 * j) % vocab for j in range(24 + 16 * i)] for i in range(4)]
        arrivals = {0: 0, 2: 1, 4: 2, 6: 3}
        step, first, finish = 0, {}, {}
        t0 = time.perf_counter()
        while step in arrivals or engine.has_unfinished() or step <= max(arrivals):
            if step in arrivals:
                engine.submit(prompts[arrivals[step]], _params(ns, max_new, stop=eos), request_id=arrivals[step])
            for o in engine.step():
                if o.token is not None:
                    first.setdefault(o.request_id, step)
                if o.finished:
                    finish[o.request_id] = step
            step += 1
        torch.cuda.synchronize()
        total = time.perf_counter() - t0
        print("request  arrival  first-token step  finish step  generated", file=out)
        generated = 0
        for step_no, rid in sorted(arrivals.items()):
            res = engine.output_of(rid)
            generated += len(res.generated_tokens)
            print(f"{rid:7d}  {step_no:7d}  {first.get(rid, -1):16d}  {finish.get(rid, -1):11d}  "
                  f"{len(res.generated_tokens):9d}", file=out)
        s = engine.scheduler.stats
        print(f"steps: {s['steps']}, tokens run: {s['tokens']}, preemptions: {s['preemptions']}", file=out)
        print(f"total: {total * 1e3:.1f} ms ({_rate(generated, total):.1f} generated tok/s)", file=out)
        return 0
    return 1


if __name__ == "__main__":
    sys.exit(main())
