"""Command line in the manner of the reference's `herbert-cli` (crates/cli/src/main.rs:54-195).

Options that exist there keep their names, meanings and defaults: --model, --backend (auto | name |
help), --max-tokens (2048), --temperature (0.4; 0 = greedy), --top-k (40; 0 = off), --top-p (0.9;
1.0 = off), --ignore-eos, --no-repeat-check, --verbose.  The reference turns --prompt text into ids
with a tokenizer; tokenizers are outside this library, so prompts are given as ids (the reference's
own fallback when no tokenizer is loaded: comma-separated ids, crates/cli/src/token_parser.rs:13-21).
Several --prompt-ids form one batch of sequences that start together.

Output: one line per sequence with its generated ids, comma-separated, in the order of the prompts.
"""

from __future__ import annotations

import argparse
import json
import sys
import tempfile
from typing import List, Optional


def parse_ids(text: str) -> List[int]:
    """Comma- or space-separated token ids."""
    try:
        ids = [int(p) for p in text.replace(",", " ").split()]
    except ValueError as e:
        raise ValueError(f"prompt ids must be integers: {e}") from None
    if not ids:
        raise ValueError("a prompt needs at least one token id")
    return ids


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="herbert-cli", description="Herbert on B200 - generation from token ids")
    ap.add_argument("--model", help="Model directory (config.json + model.safetensors)")
    ap.add_argument("--backend", default="auto", help="Backend name (default: auto; use --backend help to list options)")
    ap.add_argument("--prompt-ids", action="append", default=[], metavar="IDS",
                    help="Prompt as comma-separated token ids (repeatable: one per sequence of the batch)")
    ap.add_argument("--prompt-ids-file", help="File with one prompt per line (comma- or space-separated ids)")
    ap.add_argument("--prompt", help=argparse.SUPPRESS)
    ap.add_argument("--max-tokens", type=int, default=2048, help="Max tokens to generate (default: 2048)")
    ap.add_argument("--ignore-eos", action="store_true", help="Ignore EOS token (force generation up to max-tokens)")
    ap.add_argument("--no-repeat-check", action="store_true", help="Disable repetition loop detection")
    ap.add_argument("--stop-token-id", type=int, action="append", default=None,
                    help="Stop token id (repeatable; default: eos_token_id of config.json)")
    ap.add_argument("--verbose", action="store_true", help="Show stats after generation")
    ap.add_argument("--temperature", type=float, default=0.4, help="Sampling temperature (0 = greedy argmax)")
    ap.add_argument("--top-k", type=int, default=40, help="Top-k sampling (0 = disabled)")
    ap.add_argument("--top-p", type=float, default=0.9, help="Top-p / nucleus sampling (1.0 = disabled)")
    ap.add_argument("--seed", type=int, default=None, help="Sampling seed (default: from the clock)")
    ap.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                    help="Make random weights from --config and SEED instead of loading --model")
    ap.add_argument("--config", help="config.json for --random-weights")
    ap.add_argument("--prefill-chunk-size", type=int, default=None,
                    help="Prefill chunk size (split long prefills into chunks of N tokens)")
    ap.add_argument("--round-weights-to-bf16", action="store_true",
                    help="Round every float tensor (norm weights too) to bfloat16 while loading, as the reference does")
    ap.add_argument("--max-batch", type=int, default=None, help="Most sequences generated together")
    ap.add_argument("--max-context", type=int, default=None, help="Most positions per sequence (default: what the prompts and --max-tokens need)")
    ap.add_argument("--logits-out", help="Write the logits at each prompt's last token to this file (float32, [prompts, vocab])")
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    import herbert_rs_b200 as hb

    if args.backend == "help":
        print(hb.available_backends_help())
        return 0
    try:
        if args.prompt is not None:
            raise hb.RequestError("--prompt needs a tokenizer, which this library does not have: give --prompt-ids")
        prompts = [parse_ids(p) for p in args.prompt_ids]
        if args.prompt_ids_file:
            with open(args.prompt_ids_file) as f:
                prompts += [parse_ids(line) for line in f if line.strip()]
        if not prompts:
            raise hb.RequestError("no prompt: give --prompt-ids or --prompt-ids-file")
        backend = hb.resolve_backend(args.backend)
        tmp = None
        model_dir = args.model
        if args.random_weights is not None:
            if not args.config:
                raise hb.RequestError("--random-weights needs --config FILE")
            tmp = tempfile.TemporaryDirectory()
            model_dir = hb.write_random_model(hb.read_config_json(args.config), tmp.name, seed=args.random_weights)
        if not model_dir:
            raise hb.RequestError("--model DIR is required (or --random-weights SEED --config FILE)")
        per_seq = max(len(p) for p in prompts) + args.max_tokens
        if args.max_context is not None:
            per_seq = min(per_seq, args.max_context)
        width = min(len(prompts), args.max_batch or len(prompts))
        ps = hb.Engine.default_page_size()
        engine = hb.Engine.from_folder(model_dir, dtype=backend.dtype, max_tokens=hb.Engine.pages_for(per_seq, width) * ps,
                                       max_slots=width, max_seq_len=args.max_context,
                                       round_weights_to_bf16=args.round_weights_to_bf16)
        if args.logits_out:
            slots = [engine.alloc_slot() for _ in prompts[:width]]
            logits = engine.step(list(zip(slots, prompts[:width])), "last").cpu().numpy()
            logits.astype("<f4").tofile(args.logits_out)
            for s in slots:
                engine.free_slot(s)
        result = hb.generate(
            engine, prompts,
            hb.GenerationOptions(max_tokens=args.max_tokens, stop_token_ids=args.stop_token_id,
                                 ignore_eos=args.ignore_eos, repeat_check=not args.no_repeat_check, max_batch=width,
                                 prefill_chunk_size=args.prefill_chunk_size),
            hb.SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, seed=args.seed))
        if tmp is not None:
            tmp.cleanup()
    except (hb.HerbertError, ValueError, OSError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    for toks in result.tokens:
        print(",".join(str(t) for t in toks))
    if args.verbose:
        st = result.stats
        print(json.dumps({
            "backend": backend.name, "prompt_tokens": st.prompt_tokens, "generated_tokens": st.generated_tokens,
            "prefill_tok_s": round(st.prefill_tokens_per_second, 1), "decode_tok_s": round(st.decode_tokens_per_second, 1),
            "batches": st.batches, "finish_reasons": result.finish_reasons}), file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
