"""The Hugging Face shim: a random-init Llama-class model whose decode steps run through the
sparse decode step (the caller side of the path, twilight/pyimpl/attention.py:351-418)."""
import copy

import pytest
import torch

transformers = pytest.importorskip("transformers")
from transformers import LlamaConfig, LlamaForCausalLM  # noqa: E402

from twilight_b200 import _lib  # noqa: E402
from twilight_b200.pyimpl.hf import enable_sparse_attention  # noqa: E402

QUEST_TWI = {"selector": {"type": "quest", "token_budget": 256, "chunk_size": 16},
             "weight_estimator": {"type": "min_max_quant", "quant_bit": 4},
             "weight_pruner": {"type": "top_p", "threshold": 0.95}}
KEEP_ALL = {"selector": {"type": "none"}, "weight_estimator": {"type": "min_max_quant", "quant_bit": 4},
            "weight_pruner": {"type": "none"}, "skip_first_two_layers": False}


def _tiny_llama(layers=4):
    cfg = LlamaConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=layers,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=1024)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg).eval()


def test_prefill_is_untouched_and_decode_needs_the_cuda_library():
    model = _tiny_llama(3)
    ids = torch.randint(0, 512, (2, 40), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = model(ids, use_cache=True).logits
    info = enable_sparse_attention(model, QUEST_TWI, enable_budget_info=True)
    assert info is model.twilight_attention.budget_info and info is not None
    with torch.no_grad():
        out = model(ids, use_cache=True)
    assert (out.logits - want).abs().max() < 1e-3
    with pytest.raises(_lib.TwilightError):   # no CPU path behind the decode step
        with torch.no_grad():
            model(ids[:, :1], past_key_values=out.past_key_values, use_cache=True)


def test_head_dim_other_than_128_is_refused():
    cfg = LlamaConfig(vocab_size=64, hidden_size=128, intermediate_size=256, num_hidden_layers=1,
                      num_attention_heads=2, num_key_value_heads=2, max_position_embeddings=64)
    with pytest.raises(_lib.TwilightError):
        enable_sparse_attention(LlamaForCausalLM(cfg), KEEP_ALL)


def _decode(model, ids, steps, tokens=None):
    """Prefill + `steps` decode steps; returns per-step logits and the tokens fed."""
    logits, fed = [], []
    with torch.no_grad():
        out = model(ids, use_cache=True)
        nxt = out.logits[:, -1].argmax(-1, keepdim=True)
        for s in range(steps):
            tok = nxt if tokens is None else tokens[s]
            fed.append(tok)
            out = model(tok, past_key_values=out.past_key_values, use_cache=True)
            logits.append(out.logits[:, -1].float())
            nxt = logits[-1].argmax(-1, keepdim=True)
    return logits, fed


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_decode_with_every_token_kept_matches_the_dense_model(dt):
    dense = _tiny_llama().to("cuda", dt)
    sparse = copy.deepcopy(dense)
    enable_sparse_attention(sparse, KEEP_ALL, max_len=512)
    ids = torch.randint(0, 512, (2, 203), generator=torch.Generator().manual_seed(2)).cuda()
    want, fed = _decode(dense, ids, 20)
    got, _ = _decode(sparse, ids, 20, tokens=fed)       # 203 -> 223 tokens: crosses a page boundary
    for w, g in zip(want, got):
        assert torch.isfinite(g).all()
        assert (w - g).abs().max() <= 3e-2 * max(1.0, float(w.abs().max()))
    assert int(sparse.twilight_attention.attn._workspace(sparse.twilight_attention.caches[0].view).status.item()) == 0


@pytest.mark.gpu
def test_quest_twi_decode_records_budgets_and_stays_close_to_dense():
    dense = _tiny_llama().to("cuda", torch.bfloat16)
    sparse = copy.deepcopy(dense)
    info = enable_sparse_attention(sparse, QUEST_TWI, enable_budget_info=True, max_len=1024)
    ids = torch.randint(0, 512, (2, 600), generator=torch.Generator().manual_seed(3)).cuda()
    want, fed = _decode(dense, ids, 6)
    got, _ = _decode(sparse, ids, 6, tokens=fed)
    for w, g in zip(want, got):
        assert torch.isfinite(g).all()
    # one entry per decode step, layers 2 and 3 only (the first two layers stay dense), budgets
    # between 1 and the 256 tokens Quest passes on
    per_query = info._budget_num
    assert len(per_query) == 6
    for q in per_query:
        assert sorted(q.keys()) == [2, 3]
        for b in q.values():
            assert b.numel() == 2 * 4 and int(b.min()) >= 1 and int(b.max()) <= 256
    assert 1.0 <= info.get_total_avg_budget() <= 256.0
    # a second prompt on the same model starts over
    _decode(sparse, ids[:, :100], 2)
    assert sparse.twilight_attention.caches[0].length == 102


@pytest.mark.gpu
def test_top_p_decode_stays_close_to_dense():
    """Quest with a budget above the context keeps every page, top-p 0.95 then drops at most 5 % of
    each head's attention mass: the logits stay close to the dense model's."""
    dense = _tiny_llama().to("cuda", torch.bfloat16)
    sparse = copy.deepcopy(dense)
    cfg = copy.deepcopy(QUEST_TWI)
    cfg["selector"]["token_budget"] = 1024
    info = enable_sparse_attention(sparse, cfg, enable_budget_info=True, max_len=1024)
    ids = torch.randint(0, 512, (2, 600), generator=torch.Generator().manual_seed(4)).cuda()
    want, fed = _decode(dense, ids, 4)
    got, _ = _decode(sparse, ids, 4, tokens=fed)
    for w, g in zip(want, got):
        cos = torch.nn.functional.cosine_similarity(w, g, dim=-1)
        assert float(cos.min()) > 0.99
    assert info.get_total_avg_budget() < 604     # something was pruned
