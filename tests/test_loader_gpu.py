"""Converted checkpoints on the GPU: a small Hugging Face-style Llama / LlamaLadder checkpoint
(safetensors + config.json written by the test) is loaded through gpt_fast.loader into the drop-in
ladder model, including a config that lists `ladder_layers` (some layers dense, the others ladder),
and the CUDA engine's logits are compared with the CPU oracle on the converted weights."""
import dataclasses
import json
import os

import pytest
import torch

import golden_util as gu
from oracle import ladder_oracle as lo

pytestmark = pytest.mark.gpu

DIM, LAYERS, NH, NKV, INTER, VOCAB = 256, 4, 4, 2, 512, 512


def _hf_state(seed):
    """Random weights under the Hugging Face Llama names (q/k rows in rotate-half order)."""
    g = torch.Generator().manual_seed(seed)
    hd = DIM // NH

    def w(*shape, std=0.1, mean=0.0):
        return torch.randn(*shape, generator=g) * std + mean

    sd = {"model.embed_tokens.weight": w(VOCAB, DIM, std=0.5), "lm_head.weight": w(VOCAB, DIM),
          "model.norm.weight": w(DIM, std=0.2, mean=1.0)}
    for i in range(LAYERS):
        p = f"model.layers.{i}."
        sd[p + "self_attn.q_proj.weight"] = w(NH * hd, DIM)
        sd[p + "self_attn.k_proj.weight"] = w(NKV * hd, DIM)
        sd[p + "self_attn.v_proj.weight"] = w(NKV * hd, DIM)
        sd[p + "self_attn.o_proj.weight"] = w(DIM, NH * hd)
        sd[p + "mlp.gate_proj.weight"] = w(INTER, DIM)
        sd[p + "mlp.up_proj.weight"] = w(INTER, DIM)
        sd[p + "mlp.down_proj.weight"] = w(DIM, INTER)
        sd[p + "input_layernorm.weight"] = w(DIM, std=0.2, mean=1.0)
        sd[p + "post_attention_layernorm.weight"] = w(DIM, std=0.2, mean=1.0)
    return sd


def _oracle_full(local):
    """This package's one-rank layout -> the oracle's full tensors."""
    hd = DIM // NH
    full = {"tok_embeddings": local["tok_embeddings.weight"], "output": local["output.weight"], "norm": local["norm.weight"]}
    for i in range(LAYERS):
        p = f"layers.{i}."
        qkv, w1 = local[p + "attention.wqkv.weight"], local[p + "feed_forward.w1.weight"]
        full[f"l{i}.wq"], full[f"l{i}.wk"], full[f"l{i}.wv"] = qkv[:NH * hd], qkv[NH * hd:(NH + NKV) * hd], qkv[(NH + NKV) * hd:]
        full[f"l{i}.wo"] = local[p + "attention.wo.weight"]
        full[f"l{i}.w_up"], full[f"l{i}.w_gate"] = w1[:INTER], w1[INTER:]
        full[f"l{i}.w2"] = local[p + "feed_forward.w2.weight"]
        full[f"l{i}.attention_norm"] = local[p + "attention_norm.weight"]
        full[f"l{i}.ffn_norm"] = local[p + "ffn_norm.weight"]
    return {k: v.float() for k, v in full.items()}


@pytest.mark.parametrize("ladder_layers", [None, 2, [0, 3], []])
def test_checkpoint_with_ladder_layers_runs_on_the_gpu(tmp_path, ladder_layers):
    from safetensors.torch import save_file
    import gpt_fast
    from gpt_fast import gpt_ladder_TP
    from gpt_fast.loader import hf_to_local, load_hf_checkpoint, model_args_from_hf_config

    sd = _hf_state(5)
    save_file({k: v.contiguous() for k, v in sd.items()}, str(tmp_path / "model.safetensors"))
    config = dict(model_type="llamaLadder", vocab_size=VOCAB, hidden_size=DIM, intermediate_size=INTER,
                  num_hidden_layers=LAYERS, num_attention_heads=NH, num_key_value_heads=NKV, rope_theta=500000.0,
                  rms_norm_eps=1e-5, max_position_embeddings=256)
    if ladder_layers is not None:
        config["ladder_layers"] = ladder_layers
    (tmp_path / "config.json").write_text(json.dumps(config))

    kw = model_args_from_hf_config(str(tmp_path))
    want_layers = None if ladder_layers is None else (list(range(LAYERS - ladder_layers, LAYERS))
                                                       if isinstance(ladder_layers, int) else ladder_layers)
    assert kw.get("ladder_layers") == want_layers
    gpt_ladder_TP.transformer_configs["from-checkpoint"] = kw
    with torch.device("meta"):
        model = gpt_fast.GPTLadder.from_name("from-checkpoint")
    model = model.to(dtype=torch.bfloat16).to_empty(device="cuda").eval()
    load_hf_checkpoint(model, str(tmp_path))
    B, T, NEW = 2, 20, 4
    model.setup_caches(max_batch_size=B, max_seq_length=T + NEW)

    class Cfg:
        n_head, n_local_heads, dim, intermediate_size, n_layer = NH, NKV, DIM, INTER, LAYERS

    full = _oracle_full(hf_to_local(sd, Cfg, 0, 1))
    # a config without the field is an ordinary Llama checkpoint run under the ladder schedule (all layers ladder)
    cfg = lo.OracleConfig(block_size=256, vocab_size=VOCAB, n_layer=LAYERS, n_head=NH, n_local_heads=NKV, dim=DIM,
                          intermediate_size=INTER, rope_base=500000, ladder_layers=want_layers)
    oracle = lo.OracleModel("ladder", cfg, full, 1, torch.bfloat16, B, T + NEW)
    g = torch.Generator().manual_seed(8)
    idx, pos = torch.randint(0, VOCAB, (B, T), generator=g), torch.arange(T)
    for n in range(NEW):
        with torch.no_grad():
            got = model(idx.cuda(), pos.cuda()).float().cpu()
        ref = oracle.forward(idx, pos).float()
        err = gu.rel_err(got, ref)
        assert err < 2e-2, f"ladder_layers={ladder_layers} step {n}: {err:.3e}"
        idx = ref[:, -1].argmax(-1, keepdim=True)
        pos = torch.tensor([T + n], dtype=torch.int32)
    # the mixed schedules are really different programmes: dense-only and ladder-only logits are far apart
    if ladder_layers == []:
        other = lo.OracleModel("ladder", dataclasses.replace(cfg, ladder_layers=None), full, 1, torch.bfloat16, B, T + NEW)
        x = torch.randint(0, VOCAB, (B, T), generator=torch.Generator().manual_seed(8))
        assert gu.rel_err(other.forward(x, torch.arange(T)), oracle.forward(x, torch.arange(T))) > 0.05
