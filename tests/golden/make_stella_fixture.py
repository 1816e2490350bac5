"""Generates tests/golden/stella_tiny_hf.npz with the reference's own golden method.

The reference pins its Stella path against HF transformers' Qwen2Model run in fp32 with the
causal mask replaced by a padding-only mask (phases/03-stella/golden/generate.py:43-51), then
masked mean -> L2 -> dense head -> L2 (:87-99). The real checkpoint is not available, so the same
method is applied to a random-init Qwen2 config with the Stella structure at small dims.

Run from the repo root:  python tests/golden/make_stella_fixture.py
Needs torch + transformers (CPU). The output is committed; tests only read it.
"""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))
from stella_weights import TINY, make_batch, make_weights  # noqa: E402

import transformers.models.qwen2.modeling_qwen2 as _mq  # noqa: E402
from transformers.modeling_attn_mask_utils import _prepare_4d_attention_mask as _prep4d  # noqa: E402


def _non_causal_mask(**kwargs):
    am = kwargs["attention_mask"]
    return None if am is None else _prep4d(am, dtype=kwargs["inputs_embeds"].dtype)


_mq.create_causal_mask = _non_causal_mask
from transformers import Qwen2Config, Qwen2Model  # noqa: E402

SEED_W, SEED_B = 1234, 99


def main():
    cfg = TINY
    w = make_weights(cfg, SEED_W)
    hf_cfg = Qwen2Config(vocab_size=cfg["vocab"], hidden_size=cfg["hidden"],
                         intermediate_size=cfg["intermediate"], num_hidden_layers=cfg["n_layers"],
                         num_attention_heads=cfg["n_heads"], num_key_value_heads=cfg["n_kv_heads"],
                         max_position_embeddings=cfg["max_pos"], rms_norm_eps=cfg["rms_eps"],
                         rope_theta=cfg["rope_theta"], attention_dropout=0.0, use_sliding_window=False,
                         attn_implementation="eager")
    model = Qwen2Model(hf_cfg).to(torch.float32).eval()
    sd = {"embed_tokens.weight": w["tok_embed"], "norm.weight": w["final_norm"]}
    names = {"norm1": "input_layernorm.weight", "norm2": "post_attention_layernorm.weight",
             "wq": "self_attn.q_proj.weight", "bq": "self_attn.q_proj.bias",
             "wk": "self_attn.k_proj.weight", "bk": "self_attn.k_proj.bias",
             "wv": "self_attn.v_proj.weight", "bv": "self_attn.v_proj.bias",
             "wo": "self_attn.o_proj.weight", "w_gate": "mlp.gate_proj.weight",
             "w_up": "mlp.up_proj.weight", "w_down": "mlp.down_proj.weight"}
    for i, lw in enumerate(w["layers"]):
        for k, n in names.items():
            sd[f"layers.{i}.{n}"] = lw[k]
    missing, unexpected = model.load_state_dict({k: torch.from_numpy(v) for k, v in sd.items()}, strict=False)
    assert not unexpected and all("rotary" in m for m in missing), (missing, unexpected)

    ids, cu = make_batch(cfg, SEED_B, n_seq=5, lo=3, hi=40)
    embs, hiddens = [], []
    with torch.no_grad():
        for i in range(len(cu) - 1):
            s = torch.from_numpy(ids[cu[i]:cu[i + 1]].astype(np.int64))[None]
            mask = torch.ones_like(s)
            h = model(input_ids=s, attention_mask=mask).last_hidden_state[0]
            mf = mask[0].float().unsqueeze(-1)
            pooled = (h * mf).sum(0) / mf.sum().clamp(min=1.0)
            pooled = pooled / pooled.norm(p=2).clamp(min=1e-12)
            y = pooled @ torch.from_numpy(w["head_w"]).t() + torch.from_numpy(w["head_b"])
            y = y / y.norm(p=2).clamp(min=1e-12)
            embs.append(y.numpy().astype(np.float32))
            hiddens.append(h[-1].numpy().astype(np.float32))
    out = os.path.join(os.path.dirname(__file__), "stella_tiny_hf.npz")
    np.savez_compressed(out, seed_w=SEED_W, seed_b=SEED_B, ids=ids, cu_seqlens=cu,
                        embeddings=np.stack(embs), last_token_hidden=np.stack(hiddens),
                        torch_version=torch.__version__,
                        weight_checksum=np.float64(sum(float(np.abs(v).sum()) for v in sd.values())))
    print("wrote", out, np.stack(embs).shape)


if __name__ == "__main__":
    main()
