"""The lm-eval-harness adapter (lingua_b200.evaluation.build_harness_lm, the counterpart of apps/main/eval.py:107-163)
driven by a stand-in ``lm_eval`` package: the real one is not installed here, but the adapter only relies on the
``LM`` base class and on request objects that carry ``args``."""
import sys
import types

import pytest
import torch

from lingua_b200.generation import PackedCausalTransformerGenerator, PackedCausalTransformerGeneratorArgs
from lingua_b200.models.transformer import LMTransformer, LMTransformerArgs
from lingua_b200.tokenizer import ByteTokenizer


class _Request:
    def __init__(self, *args):
        self.args = args


@pytest.fixture()
def fake_lm_eval(monkeypatch):
    pkg, api, model = types.ModuleType("lm_eval"), types.ModuleType("lm_eval.api"), types.ModuleType("lm_eval.api.model")

    class LM:
        def __init__(self):
            self._rank, self._world_size = 0, 1

    def simple_evaluate(model, tasks=None, **kw):
        """What the harness does with a model, reduced to its three request kinds."""
        out = {}
        for t in tasks or []:
            if t == "gen":
                out[t] = model.generate_until([_Request("abc", {"until": ["\n"], "temperature": 0.0}),
                                               _Request("x", {"until": ["\n"], "temperature": 0.0})])
            elif t == "ll":
                out[t] = model.loglikelihood([_Request("hello ", "world"), _Request("a", "b")])
            elif t == "roll":
                out[t] = model.loglikelihood_rolling([_Request("some text",)])
        return {"results": out}

    model.LM = LM
    pkg.api, api.model, pkg.simple_evaluate = api, model, simple_evaluate
    for name, mod in (("lm_eval", pkg), ("lm_eval.api", api), ("lm_eval.api.model", model)):
        monkeypatch.setitem(sys.modules, name, mod)
    return pkg


def _generator():
    torch.manual_seed(0)
    args = LMTransformerArgs(dim=64, n_layers=2, n_heads=4, vocab_size=258, max_seqlen=128)
    model = LMTransformer(args)
    model.init_weights()
    model.eval()
    cfg = PackedCausalTransformerGeneratorArgs(max_gen_len=6, max_tokens=256, dtype="fp32", device="cpu")
    return model, PackedCausalTransformerGenerator(cfg, model, ByteTokenizer())


def test_harness_adapter_answers_all_three_request_kinds(fake_lm_eval):
    from lingua_b200.evaluation import build_harness_lm

    model, gen = _generator()
    lm = build_harness_lm(gen)
    res = fake_lm_eval.simple_evaluate(lm, tasks=["gen", "ll", "roll"])["results"]
    assert len(res["gen"]) == 2 and all(isinstance(g, str) and "\n" not in g for g in res["gen"])
    # log-likelihood of a continuation = sum of the model's log-probabilities of its tokens given the prefix
    tok = ByteTokenizer()
    for (ll, is_greedy), (ctx, cont) in zip(res["ll"], [("hello ", "world"), ("a", "b")]):
        ids = tok.encode(ctx + cont, add_bos=True, add_eos=False)
        with torch.no_grad():
            logp = torch.log_softmax(model(torch.tensor([ids]))[0].float(), dim=-1)
        n_ctx = len(tok.encode(ctx, add_bos=False, add_eos=False))
        tgt = torch.tensor(ids[1:])
        per_tok = logp[:-1].gather(1, tgt.view(-1, 1)).squeeze(1)
        assert abs(ll - per_tok[n_ctx:].sum().item()) < 1e-3
        assert is_greedy == bool((logp[:-1].argmax(-1) == tgt)[n_ctx:].all())
    (roll,), = res["roll"]
    ids = tok.encode("some text", add_bos=True, add_eos=False)
    with torch.no_grad():
        logp = torch.log_softmax(model(torch.tensor([ids]))[0].float(), dim=-1)
    assert abs(roll - logp[:-1].gather(1, torch.tensor(ids[1:]).view(-1, 1)).sum().item()) < 1e-3
    assert gen.max_gen_len == 6  # the scoring calls restore the generation length


def test_harness_is_skipped_without_the_package(monkeypatch):
    from lingua_b200 import evaluation

    monkeypatch.setitem(sys.modules, "lm_eval", None)
    with pytest.raises(ImportError):
        evaluation.build_harness_lm(object())
