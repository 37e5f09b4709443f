"""Hugging Face Llama checkpoints -> this package's fused, sharded layout (gpt_fast/loader.py).

Pinned against transformers' own LlamaForCausalLM on CPU: a small random model's logits must be
reproduced by the oracle model that reads the converted weights, at TP 1 and 2 (the oracle sums the
ranks' partials itself), and by the drop-in module tree (load_hf_state_dict + safetensors file)."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "ladder-residual-inference_b200"))

from oracle import ladder_oracle as lo  # noqa: E402

transformers = pytest.importorskip("transformers")

DIM, LAYERS, NH, NKV, INTER, VOCAB = 256, 3, 4, 2, 512, 512


def _hf_model(tied=False):
    cfg = transformers.LlamaConfig(vocab_size=VOCAB, hidden_size=DIM, intermediate_size=INTER, num_hidden_layers=LAYERS,
                                   num_attention_heads=NH, num_key_value_heads=NKV, rope_theta=500000.0, rms_norm_eps=1e-5,
                                   max_position_embeddings=512, tie_word_embeddings=tied, attention_bias=False,
                                   mlp_bias=False)
    torch.manual_seed(3)
    model = transformers.LlamaForCausalLM(cfg).eval()
    with torch.no_grad():  # norm weights away from 1 so that a swapped norm shows
        for name, p in model.named_parameters():
            if "norm" in name:
                p.normal_(1.0, 0.2)
    return model


def _oracle_config():
    return lo.OracleConfig(block_size=512, vocab_size=VOCAB, n_layer=LAYERS, n_head=NH, n_local_heads=NKV, dim=DIM,
                           intermediate_size=INTER, rope_base=500000, norm_eps=1e-5)


class _Cfg:  # the fields hf_to_local reads from a ModelArgs
    n_head, n_local_heads, dim, intermediate_size, n_layer = NH, NKV, DIM, INTER, LAYERS


def _full_from_rank_shards(hf_sd, world):
    """Undo the sharding: the oracle wants full tensors in this package's layout and shards them itself."""
    from gpt_fast.loader import hf_to_local
    shards = [hf_to_local(hf_sd, _Cfg, r, world) for r in range(world)]
    hd = DIM // NH
    full = {"tok_embeddings": shards[0]["tok_embeddings.weight"], "output": shards[0]["output.weight"],
            "norm": shards[0]["norm.weight"]}
    for i in range(LAYERS):
        p = f"layers.{i}."
        nq, nk = NH * hd // world, NKV * hd // world
        full[f"l{i}.wq"] = torch.cat([s[p + "attention.wqkv.weight"][:nq] for s in shards])
        full[f"l{i}.wk"] = torch.cat([s[p + "attention.wqkv.weight"][nq:nq + nk] for s in shards])
        full[f"l{i}.wv"] = torch.cat([s[p + "attention.wqkv.weight"][nq + nk:] for s in shards])
        full[f"l{i}.wo"] = torch.cat([s[p + "attention.wo.weight"] for s in shards], dim=1)
        half = INTER // world
        full[f"l{i}.w_up"] = torch.cat([s[p + "feed_forward.w1.weight"][:half] for s in shards])
        full[f"l{i}.w_gate"] = torch.cat([s[p + "feed_forward.w1.weight"][half:] for s in shards])
        full[f"l{i}.w2"] = torch.cat([s[p + "feed_forward.w2.weight"] for s in shards], dim=1)
        full[f"l{i}.attention_norm"] = shards[0][p + "attention_norm.weight"]
        full[f"l{i}.ffn_norm"] = shards[0][p + "ffn_norm.weight"]
    return full


@pytest.mark.parametrize("world", [1, 2])
@pytest.mark.parametrize("tied", [False, True])
def test_converted_weights_reproduce_hugging_face_logits(world, tied):
    hf = _hf_model(tied)
    ids = torch.randint(0, VOCAB, (2, 12), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        want = hf(ids).logits
    sd = {k: v for k, v in hf.state_dict().items()}
    if tied:
        sd.pop("lm_head.weight", None)
    full = _full_from_rank_shards(sd, world)
    names = lo.make_full_weights(_oracle_config(), 0)
    assert set(full) == set(names), sorted(set(full) ^ set(names))
    oracle = lo.OracleModel("dense", _oracle_config(), full, world, torch.float32, 2, 32)
    got = oracle.forward(ids, torch.arange(12))
    err = (got - want).abs().max() / want.abs().max()
    assert err < 2e-5, err
    # a decode step on top of the cache
    nxt = torch.randint(0, VOCAB, (2, 1), generator=torch.Generator().manual_seed(6))
    with torch.no_grad():
        want2 = hf(torch.cat([ids, nxt], dim=1)).logits[:, -1]
    got2 = oracle.forward(nxt, torch.tensor([12]))[:, -1]
    assert (got2 - want2).abs().max() / want2.abs().max() < 2e-5


def test_rotary_row_order():
    """new row 2i + j of a head = old row j * hd/2 + i."""
    from gpt_fast.loader import _interleave_rotary_rows
    hd, heads = 8, 3
    w = torch.arange(heads * hd, dtype=torch.float32).view(-1, 1).repeat(1, 2)
    out = _interleave_rotary_rows(w, heads, hd)[:, 0].view(heads, hd)
    for h in range(heads):
        assert out[h].tolist() == [h * hd + j * (hd // 2) + i for i in range(hd // 2) for j in range(2)]


def test_shape_and_family_errors():
    from gpt_fast.loader import hf_to_local
    sd = _hf_model().state_dict()
    with pytest.raises(ValueError):
        hf_to_local(sd, _Cfg, 0, 3)  # heads not divisible
    with pytest.raises(ValueError):
        hf_to_local(sd, _Cfg, 0, 1, family="parallel")
