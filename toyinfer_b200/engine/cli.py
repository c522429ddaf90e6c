"""Command line, with the reference's option names and meanings where it has them
(src/options.cpp:7-45): --model_dir, --max_seq_len, --use_dedicated_prefill,
--use_multi_stream, --enable_cuda_graph, --detail_time, --bench, --temperature, --top_k,
--top_p.  Prompts are token ids, not text: the reference's tokenizer, chat template
(--thinking) and terminal REPL are not part of this library, and neither is its beam
search (--beam_size above 1 is refused).

    bin/toyinfer --model_dir DIR --max_seq_len 4096 --prompt_ids "1,2,3;4,5" --max_new_tokens 32
    bin/toyinfer --model_dir DIR --max_seq_len 8192 --bench long
    bin/toyinfer --random config.json --seed 3 --max_seq_len 8192 --bench short
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List


def _flag(v: str) -> bool:
    if v.lower() in ("1", "true", "yes", "on"):
        return True
    if v.lower() in ("0", "false", "no", "off"):
        return False
    raise argparse.ArgumentTypeError(f"expected true/false, got {v!r}")


def _prompts(text: str) -> List[List[int]]:
    """"1,2,3;4,5" or the path of a file with one prompt per line (ids separated by
    spaces or commas), or of a JSON file holding a list of lists."""
    import os
    if os.path.isfile(text):
        with open(text) as f:
            body = f.read()
        if body.lstrip().startswith("["):
            return [list(map(int, p)) for p in json.loads(body)]
        return [[int(t) for t in line.replace(",", " ").split()] for line in body.splitlines() if line.strip()]
    return [[int(t) for t in part.replace(",", " ").split()] for part in text.split(";") if part.strip()]


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="toyinfer", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model_dir", default="", help="Model dir (config.json + safetensors)")
    ap.add_argument("--random", default="", metavar="CONFIG_JSON",
                    help="instead of --model_dir: a config.json alone; weights are drawn from --seed on the device")
    ap.add_argument("--max_seq_len", type=int, default=0, help="Maximum inference context window "
                    "(0: the model's max_position_embeddings)")
    ap.add_argument("--thinking", type=_flag, default=True, help="accepted for compatibility; selects a chat "
                    "template in the reference and has no effect on token ids")
    ap.add_argument("--use_dedicated_prefill", type=_flag, default=True,
                    help="Run prompts whole in one step instead of replaying decode token by token")
    ap.add_argument("--use_multi_stream", type=_flag, default=True,
                    help="accepted for compatibility: q, k and v (and gate and up) are one fused product here, "
                         "so there is nothing left to put on side streams")
    ap.add_argument("--enable_cuda_graph", type=_flag, default=True,
                    help="Enable CUDA graph capture/replay for decode")
    ap.add_argument("--detail_time", type=_flag, default=False,
                    help="Print prefill and decode timings: device time of every step and, where steps are "
                         "plain launches (prompts; decode with --enable_cuda_graph 0), of each layer's stages")
    ap.add_argument("--bench", default="", choices=["", "short", "long"],
                    help="Bench: a 64-token (short) or 4096-token (long) synthetic prompt, one turn")
    ap.add_argument("--temperature", type=float, default=0.6)
    ap.add_argument("--top_k", type=int, default=20)
    ap.add_argument("--top_p", type=float, default=0.95)
    ap.add_argument("--beam_size", type=int, default=1, help="only 1 (no beam search)")
    ap.add_argument("--length_penalty", type=float, default=1.0, help="unused without beam search")
    # beyond the reference
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--prompt_ids", default="", help='token ids: "1,2,3;4,5" or a file')
    ap.add_argument("--max_new_tokens", type=int, default=1024)
    ap.add_argument("--max_batch", type=int, default=64)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--ignore_eos", type=_flag, default=False)
    ap.add_argument("--prefill_chunk", type=int, default=0,
                    help="feed prompts in pieces of at most this many tokens per step (0: whole prompts)")
    return ap


def detail_lines(st, report, cuda_graph: bool) -> List[str]:
    """The ``[detail]`` block in the reference's manner (src/engine_runtime.cpp:207-261): host totals
    of the generation loop, then device times summed over steps and layers.  Stages inside a step
    that was replayed from a CUDA graph cannot be timed; the reference prints N/A for them too."""
    def ms(name):
        n, total = report.get(name, (0, 0.0))
        return n, total
    out = []
    pre = st.prompt_tokens / st.prefill_seconds if st.prefill_seconds else 0.0
    dec = st.decode_seconds / st.decode_steps * 1e3 if st.decode_steps else 0.0
    out.append(f"[detail] host: prefill {st.prefill_seconds * 1e3:.1f} ms ({pre:.0f} tok/s), decode {st.decode_steps} steps, "
               f"{dec:.3f} ms/step, batches {st.batches}")
    n, t = ms("prefill_step")
    out.append(f"[detail] prefill_total={t:.3f} ms ({n} steps)")
    for stage in ("embed", "layer.attn_block", "mixer.qkv", "mixer.attention", "mixer.out", "layer.mlp_block", "head"):
        n, t = ms("prefill." + stage)
        out.append(f"[detail] prefill.{stage}={t:.3f} ms ({n} ranges)")
    n, t = ms("decode_step")
    out.append(f"[detail] decode_forward_total={t:.3f} ms ({n} steps, {t / n if n else 0.0:.3f} ms each)")
    for stage in ("layer.attn_block", "mixer.qkv", "mixer.attention", "mixer.out", "layer.mlp_block", "head"):
        n, t = ms("decode." + stage)
        if n == 0 and cuda_graph:
            out.append(f"[detail] decode.{stage}=N/A (CUDA graph enabled)")
        else:
            out.append(f"[detail] decode.{stage}={t:.3f} ms ({n} ranges)")
    n, t = ms("sample")
    out.append(f"[detail] token_sample={t:.3f} ms ({n} draws, {t / n if n else 0.0:.3f} ms each)")
    return out


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.beam_size != 1:
        print("toyinfer: beam search is not part of this library (--beam_size must be 1)", file=sys.stderr)
        return 2
    if bool(args.model_dir) == bool(args.random):
        print("toyinfer: give either --model_dir or --random CONFIG_JSON", file=sys.stderr)
        return 2
    if not args.bench and not args.prompt_ids:
        print("toyinfer: give --prompt_ids or --bench short|long", file=sys.stderr)
        return 2
    import torch
    from .. import LLM, SamplingParams

    common = dict(dtype=args.dtype, max_seq_len=args.max_seq_len or None, max_batch=args.max_batch,
                  enable_cuda_graph=args.enable_cuda_graph, use_dedicated_prefill=args.use_dedicated_prefill,
                  detail_time=args.detail_time, prefill_chunk=args.prefill_chunk or None)
    if args.random:
        with open(args.random) as f:
            llm = LLM(config=json.load(f), seed=args.seed, **common)
    else:
        llm = LLM(args.model_dir, **common)
    vocab = llm.engine.spec.vocab_size
    max_new = args.max_new_tokens
    ignore_eos = args.ignore_eos
    if args.bench:
        n = 64 if args.bench == "short" else 4096
        g = torch.Generator().manual_seed(args.seed)
        prompts = [torch.randint(0, vocab, (n,), generator=g).tolist()]
        max_new = min(max_new, 1024)          # the reference caps a bench turn at 1024 new tokens
    else:
        prompts = _prompts(args.prompt_ids)
    params = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, seed=args.seed)
    t0 = time.perf_counter()
    results = llm.generate(prompts, params, max_new_tokens=max_new, ignore_eos=ignore_eos)
    wall = time.perf_counter() - t0
    for i, r in enumerate(results):
        print(json.dumps({"request": i, "tokens": r.tokens, "finish_reason": r.finish_reason}))
    st = llm.last_stats
    total = st.prompt_tokens + st.generated_tokens
    print(f"[perf] prompt_tokens={st.prompt_tokens} generated_tokens={st.generated_tokens} "
          f"wall={wall:.3f}s tokens/s={total / wall:.2f}", file=sys.stderr)
    if args.detail_time:
        for line in detail_lines(st, llm.timing_report(), args.enable_cuda_graph):
            print(line, file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
