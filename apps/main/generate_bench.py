"""Generation throughput of the packed KV-cache generator on a random-init model.

    python -m apps.main.generate_bench [--model 1b|7b|hawk_1b|mingru_1b|minlstm_1b|mamba_1b] [--batch 32]
                                       [--prompt 512] [--new 256]

Times ``PackedCausalTransformerGenerator.generate`` (prefill of all prompts packed in one sequence, then one
decode step per new token for the whole batch; apps/main/generate.py:310-420 of the reference) with CUDA events
after one warm-up call and prints one JSON line with the end-to-end and decode-only tokens/s.
"""
from __future__ import annotations

import argparse
import json

import torch

from lingua_b200.generation import PackedCausalTransformerGenerator, PackedCausalTransformerGeneratorArgs
from lingua_b200.models.transformer import LMTransformer, LMTransformerArgs
from lingua_b200.tokenizer import build_tokenizer

MODELS = {
    "1b": dict(dim=2048, n_layers=25, n_heads=16, vocab_size=128256, max_seqlen=4096),
    "7b": dict(dim=4096, n_layers=32, n_heads=32, rope_theta=100000.0, ffn_dim_multiplier=1.0, multiple_of=256,
               vocab_size=128256, max_seqlen=4096),
}


# recurrent / state-space families: generated with the state-cache generator (lingua_b200/generation_recurrent.py)
RECURRENT = {
    "hawk_1b": ("lingua_b200.models.fastrnn", "LMHawk", "LMHawkArgs",
                dict(dim=2048, n_layers=24, n_heads=16, conv_size=4, lru_dim_multiplier=1.0, ffn_dim_multiplier=1.125,
                     vocab_size=128256)),
    "mingru_1b": ("lingua_b200.models.fastrnn", "LMMinGRU", "LMMinGRUArgs",
                  dict(dim=2048, n_layers=24, n_heads=16, conv_size=4, vocab_size=128256)),
    "minlstm_1b": ("lingua_b200.models.fastrnn", "LMMinLSTM", "LMMinLSTMArgs",
                   dict(dim=2048, n_layers=24, n_heads=16, conv_size=4, vocab_size=128256)),
    "mamba_1b": ("lingua_b200.models.mamba", "LMMamba", "LMMambaArgs",
                 dict(dim=2048, n_layers=48, n_heads=64, state_dim=128, n_groups=1, conv_size=4, ssm_chunk_size=256,
                      vocab_size=128256)),
}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="1b", choices=list(MODELS) + list(RECURRENT))
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--eager", action="store_true", help="do not replay the decode step as a CUDA graph")
    a = ap.parse_args(argv)
    dev = torch.device("cuda")
    gen_cls = PackedCausalTransformerGenerator
    torch.manual_seed(0)
    if a.model in RECURRENT:
        import importlib

        from lingua_b200.generation_recurrent import PackedRNNGenerator as gen_cls

        mod_name, cls_name, args_name, kw = RECURRENT[a.model]
        mod = importlib.import_module(mod_name)
        with torch.device(dev):
            model = getattr(mod, cls_name)(getattr(mod, args_name)(**kw))
        a.eager = True  # the state-cache step is not captured as a CUDA graph
    else:
        with torch.device(dev):
            model = LMTransformer(LMTransformerArgs(**MODELS[a.model]))
    model.init_weights()
    for p in model.parameters():
        p.data = p.data.to(torch.bfloat16)
    model.eval()
    tok = build_tokenizer("bytes")
    cfg = PackedCausalTransformerGeneratorArgs(temperature=0.0, max_gen_len=a.new, max_prompt_len=a.prompt,
                                               max_tokens=a.batch * (a.prompt + a.new),
                                               reduce_generation_overhead=not a.eager)
    gen = gen_cls(cfg, model, tok)
    g = torch.Generator().manual_seed(1)
    prompts = ["".join(chr(97 + int(c)) for c in torch.randint(0, 26, (a.prompt - 1,), generator=g)) for _ in range(a.batch)]

    def run():
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        out = gen.generate(prompts)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1), out

    run()  # warm-up: cache allocation, kernel loading
    ms, out = run()
    n_new = a.batch * a.new
    # prefill alone, to separate the decode phase
    cfg0 = PackedCausalTransformerGeneratorArgs(temperature=0.0, max_gen_len=1, max_prompt_len=a.prompt,
                                                max_tokens=a.batch * (a.prompt + 1))
    gen0 = gen_cls(cfg0, model, tok)
    gen.release_cache()
    gen0.generate(prompts)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    gen0.generate(prompts)
    e1.record()
    torch.cuda.synchronize()
    ms_prefill = e0.elapsed_time(e1)
    print(json.dumps({
        "metric": "generation tokens/s (greedy, packed prompts, KV or state cache)",
        "model": a.model if a.model in RECURRENT else f"llama_{a.model}", "batch": a.batch,
        "prompt_tokens": a.prompt, "new_tokens": a.new, "ms_total": round(ms, 1), "ms_prefill": round(ms_prefill, 1),
        "tokens_per_s_end_to_end": round(n_new / ms * 1e3, 1),
        "tokens_per_s_decode": round(n_new / max(ms - ms_prefill, 1e-3) * 1e3, 1),
        "ms_per_decode_step": round((ms - ms_prefill) / a.new, 3), "cuda_graph": not a.eager, "dtype": "bf16",
        "data": "random prompts, random-init weights"}))


if __name__ == "__main__":
    main()
