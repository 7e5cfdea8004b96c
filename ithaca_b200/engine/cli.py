"""The command line, in the manner of the reference's prompt mode (src/main.cpp:945-1144).

Options the reference has keep its names and meanings: ``--model/-m``, ``--prompt/-p``,
``-n`` (default 128), ``--temp`` (default 0), ``--ctx/-c``, ``--bench`` (prompt of 512 and
128 generated tokens, three runs after a warm-up of 64, printed as one ``BENCH`` line,
src/main.cpp:1047-1068).  ``--profile`` stands for the reference's ``ITHACA_PROF`` timers
(src/model.cpp:1261-1307): it runs the prompts as one step and then one more token each, with
CUDA events around every kernel call, and prints both steps kernel by kernel.  There is no tokenizer in this library, so a prompt is a list of
token ids (``-p "1,2,3"``); ``-p`` may be given several times for a batch.  After the run
it prints ``[prompt N tok @ X tok/s | gen M tok @ Y tok/s]`` (src/main.cpp:1140).
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List, Optional


def _ids(text: str) -> List[int]:
    try:
        return [int(x) for x in text.replace(",", " ").split()]
    except ValueError:
        raise SystemExit(f"a prompt is a list of token ids separated by commas or spaces, found {text!r}")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="ithaca_b200", description="generate tokens with a model folder on one B200")
    ap.add_argument("--model", "-m", help="folder with config.json and *.safetensors")
    ap.add_argument("--random", metavar="CONFIG.json", help="instead of --model: random weights for this configuration")
    ap.add_argument("--seed", type=int, default=0, help="seed of the random weights (--random) and of sampling")
    ap.add_argument("--prompt", "-p", action="append", default=[], help="token ids, e.g. \"1,2,3\"; repeatable")
    ap.add_argument("--prompt-file", help="a file with one prompt (token ids) per line")
    ap.add_argument("-n", type=int, default=128, dest="n", help="tokens to generate per prompt (default 128)")
    ap.add_argument("--temp", type=float, default=0.0, help="temperature; 0 = greedy (default)")
    ap.add_argument("--top-k", type=int, default=40)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--rep-pen", type=float, default=1.1, help="repetition penalty over the last 64 generated ids")
    ap.add_argument("--stop-ids", default=None, help="stop token ids (default: the model's eos_token_id)")
    ap.add_argument("--ctx", "-c", type=int, default=None, help="most positions per sequence (default: the model's)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-tokens", type=int, default=None, help="cache size in positions (default: 8 sequences of ctx)")
    ap.add_argument("--bench", action="store_true", help="pp512 / tg128, three runs, one BENCH line")
    ap.add_argument("--profile", action="store_true",
                    help="time every kernel call of a prompt step and of a decode step and print the tables")
    ap.add_argument("--peaks", metavar="FILE.json", default=None,
                    help="with --profile: hbm_gbs and bf16_tflops to hold the kernels against (default: measured now)")
    ap.add_argument("--describe", action="store_true", help="print the model's layers and schedule, then exit")
    ap.add_argument("--selftest", action="store_true",
                    help="check this installation on the device without a model folder: a small random model whole against "
                         "token by token (same bits in float32), bfloat16 against float32, the kernels' bounded waits")
    return ap


def _engine(args):
    from .api import Engine
    if args.random:
        with open(args.random) as f:
            cfg = json.load(f)
        return Engine.from_random(cfg, args.seed, dtype=args.dtype, max_tokens=args.max_tokens, ctx=args.ctx)
    if not args.model:
        raise SystemExit("give --model DIR (or --random CONFIG.json)")
    return Engine(args.model, dtype=args.dtype, max_tokens=args.max_tokens, ctx=args.ctx)


def _bench(eng, name: str, load_s: float) -> None:
    import numpy as np
    import torch
    vocab = eng.model.spec.vocab_size
    rng = np.random.default_rng(0)
    eng.generate([rng.integers(0, vocab, 64).tolist()], max_tokens=2, temp=0.0, rep_pen=1.0, stop_token_ids=[])
    pp, tg = [], []
    for _ in range(3):
        eng.generate([rng.integers(0, vocab, 512).tolist()], max_tokens=129, temp=0.0, rep_pen=1.0, stop_token_ids=[])
        st = eng.last_stats
        pp.append(512 / st.prefill_seconds)
        tg.append(128 / st.decode_seconds)
    vram = torch.cuda.max_memory_allocated() / 2**20
    print(f"BENCH model={name} load_s={load_s:.2f} pp512={sum(pp) / 3:.1f} tg128={sum(tg) / 3:.2f} vram_mb={vram:.0f}")


def _profile(eng, prompts: List[List[int]], peaks_file: Optional[str]) -> None:
    from .profile import format_table, measure_peaks
    if peaks_file:
        with open(peaks_file) as f:
            peaks = json.load(f)
    else:
        peaks = measure_peaks(eng.runtime.device)
    print(f"peaks: {peaks['hbm_gbs']} GB/s, {peaks['bf16_tflops']} TFLOP/s bfloat16"
          + (f" ({peaks['how']})" if "how" in peaks else ""))
    slots = [eng.alloc_slot() for _ in prompts]
    eng.step(slots, prompts, "last")                       # warm-up: whatever still has to be compiled or loaded
    for s in slots:
        eng.truncate(s, 0)
    logits, rows = eng.profile_step(slots, prompts, "last")
    print(format_table(rows, peaks, f"prompt step: {sum(len(p) for p in prompts)} tokens of {len(prompts)} sequences"))
    nxt = [[int(t)] for t in logits.argmax(-1).tolist()]
    eng.profile_step(slots, nxt, "last")
    _, rows = eng.profile_step(slots, nxt, "last")
    print(format_table(rows, peaks, f"decode step: one token of {len(prompts)} sequences"))
    eng.check_status()
    for s in slots:
        eng.free_slot(s)


def _selftest() -> int:
    """The reference's command line carries self-tests of its kernels (``--fatest``, ``--quanttest`` and others,
    src/main.cpp:986-1031).  This one needs no files: the model is random."""
    import torch
    from ..csrc import ops
    from .api import Engine
    cfg = {"architectures": ["LlamaForCausalLM"], "hidden_size": 264, "num_hidden_layers": 3, "num_attention_heads": 6,
           "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 520, "vocab_size": 1003, "rope_theta": 500000.0,
           "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 64},
           "rms_norm_eps": 1e-5, "max_position_embeddings": 1024, "tie_word_embeddings": True, "torch_dtype": "bfloat16"}
    ids = [(7 * i * i + 3 * i + 1) % 1003 for i in range(300)]
    failed = 0

    def report(name: str, ok: bool, detail: str) -> None:
        nonlocal failed
        failed += not ok
        print(f"{'ok  ' if ok else 'FAIL'} {name}: {detail}")

    logits = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_random(cfg, 1, dtype=dtype, max_tokens=1024)
        s = eng.alloc_slot()
        whole = eng.step([s], [ids], "all").float()
        eng.free_slot(s)
        s = eng.alloc_slot()
        rows = [eng.step([s], [ids[:130]], "all").float()] + [eng.step([s], [ids[130:261]], "all").float()]
        rows += [eng.step([s], [[t]], "last").float() for t in ids[261:]]
        eng.check_status()
        cut = torch.cat(rows)
        diff = float((cut - whole).abs().max() / whole.abs().max())
        report(f"{dtype}: two pieces and 39 single tokens against the whole prompt", diff == 0.0 if dtype == "float32" else diff <= 1e-2,
               f"largest difference {diff:.3g} of the logits' scale")
        out = eng.generate([ids[:40], ids[:7]], max_tokens=12, temp=0.0, rep_pen=1.0, stop_token_ids=[])
        report(f"{dtype}: greedy generation of two requests", all(len(o) == 12 for o in out), f"{out[1]}")
        logits[dtype] = whole
    diff = float((logits["bfloat16"] - logits["float32"]).abs().max() / logits["float32"].abs().max())
    report("bfloat16 against float32", diff <= 2e-2, f"largest difference {diff:.3g} of the logits' scale")
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    res = ops.selftest_wait_expires(status, 1_000_000).cpu().tolist()
    report("a wait that nothing satisfies gives up", res[0] == 0 and res[1] == 1 and res[3] == 0 and res[5] == 0 and int(status.item()) == 8,
           f"after {res[2]} us; a second waiter left after {res[4]} us")
    print("selftest passed" if not failed else f"selftest: {failed} check(s) FAILED")
    return 1 if failed else 0


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    if args.selftest:
        return _selftest()
    t0 = time.perf_counter()
    eng = _engine(args)
    load_s = time.perf_counter() - t0
    spec = eng.model.spec
    print(f"[{args.model or args.random} | {spec.architecture} | {len(spec.schedule)} layers | {args.dtype} | "
          f"opened in {load_s * 1e3:.0f} ms]", file=sys.stderr)
    if args.describe:
        from ..config import describe
        print("\n".join(describe(spec)))
        return 0
    if args.bench:
        _bench(eng, args.model or args.random, load_s)
        return 0
    prompts = [_ids(p) for p in args.prompt]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [_ids(line) for line in f if line.strip()]
    if not prompts:
        raise SystemExit("give at least one --prompt (token ids)")
    if args.profile:
        _profile(eng, prompts, args.peaks)
        return 0
    stops = _ids(args.stop_ids) if args.stop_ids is not None else None
    out = eng.generate(prompts, max_tokens=args.n, temp=args.temp, top_k=args.top_k, top_p=args.top_p,
                       rep_pen=args.rep_pen, seed=args.seed, stop_token_ids=stops)
    for o in out:
        print(",".join(str(t) for t in o))
    st = eng.last_stats
    print(f"[prompt {st.prompt_tokens} tok @ {st.prefill_tps:.1f} tok/s | gen {st.gen_tokens} tok @ {st.gen_tps:.1f} tok/s]",
          file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
