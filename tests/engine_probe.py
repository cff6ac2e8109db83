"""Runs one engine configuration in a fresh process and prints the generated token ids as
JSON (used by multi-GPU tests so that every configuration gets fresh processes on all ranks)."""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--dp", type=int, default=1)
    ap.add_argument("--comm", default="auto")
    ap.add_argument("--cg", action="store_true")
    ap.add_argument("--port", type=int, default=29811)
    ap.add_argument("--max-tokens", type=int, default=10)
    ap.add_argument("--prefix-backend", default="hash")
    ap.add_argument("--prompt-lens", default="5,16,40,100")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--pp-microbatches", type=int, default=1)
    a = ap.parse_args()
    import torch

    from xixi_vllm_b200 import Engine, EngineConfig, SamplingParams
    g = torch.Generator().manual_seed(0)
    cfg = EngineConfig(model=a.model, dtype="bfloat16", num_kvcache_blocks=256, max_num_seqs=16,
                       max_num_batched_tokens=256, context_len=512, tp_size=a.tp, pp_size=a.pp, dp_size=a.dp,
                       tp_comm=a.comm, enforce_eager=not a.cg, nccl_port=a.port, prefix_backend=a.prefix_backend,
                       pp_microbatches=a.pp_microbatches)
    vocab = cfg.hf_config.vocab_size
    prompts = [torch.randint(0, vocab, (int(n),), generator=g).tolist() for n in a.prompt_lens.split(",")]
    eng = Engine(cfg)
    try:
        sp = SamplingParams(max_tokens=a.max_tokens, ignore_eos=True, temperature=a.temperature,
                            top_k=20 if a.temperature > 0 else None)
        seqs = [eng.add_request(p, sp) for p in prompts]
        while eng.has_unfinished():
            eng.step()
        out = [s.token_ids[s.num_prompt_tokens:] for s in seqs]
    finally:
        eng.destroy()
    print("RESULT " + json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
