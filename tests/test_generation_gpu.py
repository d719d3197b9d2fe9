"""Native generation path: packed prefill + KV-cache decode kernel vs a full forward pass."""
import pytest
import torch

from lingua_b200.generation import PackedCausalTransformerGenerator, PackedCausalTransformerGeneratorArgs
from lingua_b200.models.transformer import LMTransformer, LMTransformerArgs
from lingua_b200.tokenizer import ByteTokenizer

pytestmark = pytest.mark.gpu


def test_prefill_and_decode_match_full_forward():
    torch.manual_seed(0)
    args = LMTransformerArgs(dim=512, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=258, max_seqlen=256)
    model = LMTransformer(args)
    model.init_weights()
    model = model.cuda().bfloat16().eval()
    model.rope_embeddings.reset_parameters()
    tok = ByteTokenizer()
    gen = PackedCausalTransformerGenerator(PackedCausalTransformerGeneratorArgs(max_gen_len=8, max_tokens=512), model, tok)
    prompts = ["hello world, this is a test", "abc", "the quick brown fox jumps over"]
    ids = [tok.encode(p, add_bos=True) for p in prompts]
    with torch.inference_mode():
        # reference: every prompt alone through the plain forward
        full = [model(torch.tensor([i], device="cuda")).float()[0] for i in ids]
        packed = torch.cat([torch.tensor(i[:-1]) for i in ids]).cuda()
        lengths = torch.tensor([len(i) - 1 for i in ids]).cuda()
        pre = gen.prefill(packed.unsqueeze(0), lengths).float()[0]
        last = torch.tensor([[i[-1] for i in ids]], device="cuda")
        nxt = gen.generate_next_token(last).float()[0]
        gen.release_cache()
    off = 0
    for k, i in enumerate(ids):
        n = len(i) - 1
        ref = full[k]
        scale = ref.abs().max().item()
        assert (pre[off:off + n] - ref[:n]).abs().max().item() < 4e-2 * scale
        assert (nxt[k] - ref[n]).abs().max().item() < 4e-2 * scale
        off += n


def test_generate_api_runs_greedy():
    torch.manual_seed(1)
    args = LMTransformerArgs(dim=256, n_layers=2, n_heads=2, vocab_size=258, max_seqlen=128)
    model = LMTransformer(args)
    model.init_weights()
    model = model.cuda().bfloat16().eval()
    model.rope_embeddings.reset_parameters()
    gen = PackedCausalTransformerGenerator(PackedCausalTransformerGeneratorArgs(max_gen_len=6, max_tokens=256), model,
                                           ByteTokenizer())
    texts, lls, greedy = gen.generate(["first prompt", "second"])
    assert len(texts) == 2 and len(lls[0]) == len("first prompt") and all(torch.isfinite(l).all() for l in lls)


def test_graph_replayed_decode_matches_eager():
    torch.manual_seed(2)
    args = LMTransformerArgs(dim=256, n_layers=2, n_heads=2, vocab_size=258, max_seqlen=128)
    model = LMTransformer(args)
    model.init_weights()
    model = model.cuda().bfloat16().eval()
    model.rope_embeddings.reset_parameters()
    prompts = ["a first prompt", "second", "and a third one"]
    outs = []
    for graph in (False, True):
        gen = PackedCausalTransformerGenerator(
            PackedCausalTransformerGeneratorArgs(max_gen_len=12, max_tokens=512, reduce_generation_overhead=graph),
            model, ByteTokenizer())
        outs.append(gen.generate(prompts)[0])
        outs.append(gen.generate(prompts[:2])[0])  # second call: new batch shape, graph is rebuilt
    assert outs[0] == outs[2] and outs[1] == outs[3]
