"""Checkpoint loading on the GPU: a Stella-structure checkpoint directory written with the
`safetensors` package loads through the native loader into the same model as the in-memory
constructor (bit-identical embeddings), with the reference's tensor accounting errors
(crates/encoders/src/stella.rs:126-145, :376-400; crates/embed/src/stella.rs:380-443); the device
quantiser reproduces the CPU definition bit for bit; the decoder loads from a Qwen2-style file."""
import os

import numpy as np
import pytest
import torch

import oracle_lib as O
from gpu_util import DEV, TOL, max_rel
from logismos_b200._lib import lib
from logismos_b200.decoder import BlockAllocator, DecoderModel
from logismos_b200.embed import ComputeError, EncodeOpts, IoError, StellaModel
from logismos_b200.loader import quantize_int4
from logismos_b200.text import Prompt, StellaTextModel
from stella_weights import TINY, make_batch, make_weights, quantize_weights
from test_loader_text import make_tokenizer

pytestmark = pytest.mark.gpu

NAMES = {"norm1": "input_layernorm.weight", "norm2": "post_attention_layernorm.weight", "wq": "self_attn.q_proj.weight",
         "bq": "self_attn.q_proj.bias", "wk": "self_attn.k_proj.weight", "bk": "self_attn.k_proj.bias", "wv": "self_attn.v_proj.weight",
         "bv": "self_attn.v_proj.bias", "wo": "self_attn.o_proj.weight", "w_gate": "mlp.gate_proj.weight", "w_up": "mlp.up_proj.weight",
         "w_down": "mlp.down_proj.weight"}


def tensors_of(w):
    t = {"model.embed_tokens.weight": w["tok_embed"], "model.norm.weight": w["final_norm"]}
    for i, lw in enumerate(w["layers"]):
        for k, n in NAMES.items():
            t[f"model.layers.{i}.{n}"] = lw[k]
    return t


def write_checkpoint(root, w, heads):
    from safetensors.numpy import save_file
    os.makedirs(root, exist_ok=True)
    save_file(tensors_of(w), os.path.join(root, "model.safetensors"))
    for d, (hw, hb) in heads.items():
        os.makedirs(os.path.join(root, f"2_Dense_{d}"), exist_ok=True)
        save_file({"linear.weight": hw, "linear.bias": hb}, os.path.join(root, f"2_Dense_{d}", "model.safetensors"))


def test_stella_checkpoint_loads_into_the_same_model(tmp_path):
    w = make_weights(TINY, 1234)
    rng = np.random.default_rng(3)
    heads = {128: (w["head_w"], w["head_b"]), 64: ((rng.standard_normal((64, TINY["hidden"])) * 0.02).astype(np.float32),
                                                   (rng.standard_normal(64) * 0.02).astype(np.float32))}
    root = str(tmp_path / "ckpt")
    write_checkpoint(root, w, heads)
    ids, cu = make_batch(TINY, 5, n_seq=4, lo=3, hi=60)
    lib.logismos_set_deterministic(1)   # fixed summation order: equal weights must give bit-identical embeddings
    ref = StellaModel(TINY, w, max_batch_tokens=256, max_batch_seqs=8, heads=heads)
    got = StellaModel.load(root, dims=[128, 64], cfg=TINY, max_batch_tokens=256, max_batch_seqs=8)
    assert got.supported_dims() == [64, 128] or sorted(got.supported_dims()) == [64, 128]
    assert got.default_dim() == 64   # no 1024 head: the smallest loaded dim is the default
    for dim in (64, 128):
        assert np.array_equal(got.encode_ids_batch(ids, cu, EncodeOpts(dim=dim)), ref.encode_ids_batch(ids, cu, EncodeOpts(dim=dim)))
    got.close(); ref.close()
    # the text model over the same directory: tokenizer.json + prompt sidecar
    make_tokenizer(os.path.join(root, "tokenizer.json"), [f"w{i}" for i in range(200)])
    open(os.path.join(root, "config_sentence_transformers.json"), "w").write('{"prompts": {"s2s_query": "w1 w2 "}}')
    tm = StellaTextModel.load(root, dims=[128], cfg=TINY, max_batch_tokens=256, max_batch_seqs=8)
    e = tm.encode_batch(["w5 w6 w7", "w9"], EncodeOpts(prompt=Prompt.s2s_query()))
    assert e.shape == (2, 128) and np.allclose(np.linalg.norm(e, axis=1), 1.0, atol=1e-5)
    direct = tm.model.encode_ids_batch(np.array([3, 4, 7, 8, 9, 1, 3, 4, 11, 1], np.uint32), np.array([0, 6, 10], np.int32))
    assert np.array_equal(e, direct)
    # with the switch on a sequence encoded alone equals its row in the batch, bit for bit
    alone = tm.model.encode_ids_batch(np.array([3, 4, 11, 1], np.uint32), np.array([0, 4], np.int32))
    assert np.array_equal(alone[0], e[1])
    tm.model.close()
    lib.logismos_set_deterministic(0)


def test_stella_loader_accounts_for_every_tensor(tmp_path):
    from safetensors.numpy import save_file
    w = make_weights(TINY, 7)
    heads = {128: (w["head_w"], w["head_b"])}
    root = str(tmp_path / "ckpt")
    write_checkpoint(root, w, heads)
    t = tensors_of(w)
    path = os.path.join(root, "model.safetensors")

    def load():
        return StellaModel.load(root, dims=[128], cfg=TINY, max_batch_tokens=64, max_batch_seqs=2)

    short = dict(t); del short["model.layers.1.mlp.up_proj.weight"]
    save_file(short, path)
    with pytest.raises(ComputeError, match="expected 26 tensors in stella archive, got 25"):
        load()
    extra = dict(t); extra["rogue"] = np.zeros(1, np.float32)
    save_file(extra, path)
    with pytest.raises(ComputeError, match="got 27"):
        load()
    renamed = dict(t); renamed["model.layers.0.self_attn.qq_proj.weight"] = renamed.pop("model.layers.0.self_attn.q_proj.weight")
    save_file(renamed, path)
    with pytest.raises(Exception, match="tensor not found: model.layers.0.self_attn.q_proj.weight"):
        load()
    shaped = dict(t); shaped["model.layers.0.self_attn.k_proj.weight"] = np.zeros((TINY["hidden"], 256), np.float32)
    save_file(shaped, path)
    with pytest.raises(ComputeError, match=r"expected shape \[256, 512\], got \[512, 256\]"):
        load()
    typed = dict(t); typed["model.norm.weight"] = typed["model.norm.weight"].astype(np.float16)
    save_file(typed, path)
    with pytest.raises(ComputeError, match="model.norm.weight: expected F32"):
        load()
    save_file(t, path)
    save_file({"linear.weight": w["head_w"][:, :100].copy(), "linear.bias": w["head_b"]}, os.path.join(root, "2_Dense_128", "model.safetensors"))
    with pytest.raises(IoError, match="dense head 2_Dense_128: expected weight shape"):
        load()
    with pytest.raises(IoError):
        StellaModel.load(root, dims=[256], cfg=TINY)   # no such head directory


def test_device_quantiser_is_bit_exact_and_decoder_loads_from_a_checkpoint(tmp_path):
    from safetensors.numpy import save_file
    rng = np.random.default_rng(11)
    m = (rng.standard_normal((96, 256)) * 0.05).astype(np.float32)
    m[3, 32:64] = 0.0                      # an all-zero group: scale 0, codes 0
    m[5, 0] = 7.5 * np.abs(m[5, :32]).max()  # values that round at .5
    codes, scales = quantize_int4(torch.from_numpy(m).to(DEV))
    ref_c, ref_s = O.int4_quantize(m)
    assert np.array_equal(codes.cpu().numpy(), ref_c) and np.array_equal(scales.cpu().numpy().view(np.uint16), np.asarray(ref_s).view(np.uint16))
    # decoder: fp32 Qwen2-style file -> native loader (quantises on the device) == in-memory int4 weights quantised by the oracle
    w = make_weights(TINY, 77)
    qw, deq = quantize_weights(TINY, w)
    t = tensors_of(w)
    lm = np.random.Generator(np.random.PCG64(5)).standard_normal((TINY["vocab"], TINY["hidden"]), dtype=np.float32) * np.float32(0.02)
    t["lm_head.weight"] = lm     # the same draw quantize_weights uses for its head
    path = str(tmp_path / "decoder.safetensors")
    save_file(t, path)
    lib.logismos_set_deterministic(1)
    a = DecoderModel(TINY, qw, n_pool_blocks=16, max_blocks_per_seq=8, max_step_tokens=128, max_step_seqs=2)
    b = DecoderModel.load(path, TINY, n_pool_blocks=16, max_blocks_per_seq=8, max_step_tokens=128, max_step_seqs=2)
    alloc = BlockAllocator(16, 8, seed=1)
    ids = rng.integers(0, TINY["vocab"], 50)
    tab = alloc.ensure(0, 50)[None, :]
    ta, tb = a.step(ids, [0], [50], tab), b.step(ids, [0], [50], tab)
    assert np.array_equal(ta, tb) and np.array_equal(a.last_logits(), b.last_logits())
    h = O.OracleStella(TINY, deq).forward(ids.astype(np.uint32), causal=True)[-1]
    assert max_rel(b.last_hidden()[0], h) <= TOL
    a.close(); b.close()
    del t["lm_head.weight"]      # tied head: the embedding doubles as lm_head
    save_file(t, path)
    c = DecoderModel.load(path, TINY, n_pool_blocks=16, max_blocks_per_seq=8, max_step_tokens=128, max_step_seqs=2)
    c.step(ids, [0], [50], tab)
    assert c.device_status() == 0
    c.close()
    lib.logismos_set_deterministic(0)
