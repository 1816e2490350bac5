"""The sampling chain on device logits: the Python mirror of the reference's decode crate
(crates/decode/src/{chain,processors,sampler}.rs) over the C ABI. A chain is a list of processors
followed by one sampler; processors mutate fp32 CUDA logits [rows, vocab] in place, in insertion
order, and the sampler returns one token id per row. Nothing leaves the device except the tokens.

    chain = DecodeChain(MultinomialSampler(seed=7)).push(TemperatureScale(0.8)).push(TopK(50)).push(TopP(0.95))
    tokens = chain.step(logits)            # uint32 CUDA tensor [rows]
"""
from __future__ import annotations

import torch

from ._lib import check, lib
from .ops import InvalidOp, _p, _stream


def _rows(logits):
    if not isinstance(logits, torch.Tensor) or not logits.is_cuda:
        raise InvalidOp("sampling: logits must be a CUDA tensor (there is no CPU arm)")
    if logits.dtype != torch.float32 or logits.dim() != 2 or not logits.is_contiguous():
        raise InvalidOp("sampling: logits must be contiguous fp32 [rows, vocab]")
    return logits.shape


class TemperatureScale:
    """processors.rs:15-28."""

    def __init__(self, temperature: float):
        self.t = float(temperature)

    def process(self, logits, ctx=None):
        r, n = _rows(logits)
        check(lib.logismos_launch_temperature_f32(_p(logits), r, n, self.t, _stream()), "temperature")


class TopK:
    """processors.rs:30-82."""

    def __init__(self, k: int):
        self.k = int(k)

    def process(self, logits, ctx=None):
        r, n = _rows(logits)
        check(lib.logismos_launch_top_k_f32(_p(logits), r, n, self.k, _stream()), "top_k")


class TopP:
    """processors.rs:84-122."""

    def __init__(self, p: float):
        self.p = float(p)

    def process(self, logits, ctx=None):
        r, n = _rows(logits)
        check(lib.logismos_launch_top_p_f32(_p(logits), r, n, self.p, _stream()), "top_p")


class MinP:
    """processors.rs:124-146."""

    def __init__(self, p: float):
        self.p = float(p)

    def process(self, logits, ctx=None):
        r, n = _rows(logits)
        check(lib.logismos_launch_min_p_f32(_p(logits), r, n, self.p, _stream()), "min_p")


class RepetitionPenalty:
    """processors.rs:148-181. ``tokens``: uint32 CUDA tensor [rows, max_tokens] (int32 accepted), ``counts``:
    int32 CUDA tensor [rows] of how many entries of each row are live."""

    def __init__(self, tokens, counts, penalty: float):
        self.tokens, self.counts, self.penalty = tokens, counts, float(penalty)

    def process(self, logits, ctx=None):
        r, n = _rows(logits)
        t, c = self.tokens, self.counts
        if not (t.is_cuda and c.is_cuda) or t.dim() != 2 or t.shape[0] != r or c.shape != (r,) or c.dtype != torch.int32 or t.element_size() != 4:
            raise InvalidOp("repetition_penalty: tokens [rows, max] (32-bit) and counts int32 [rows] on the device")
        check(lib.logismos_launch_repetition_penalty_f32(_p(logits), r, n, _p(t.contiguous()), _p(c), t.shape[1], self.penalty, _stream()),
              "repetition_penalty")


class TypicalSampling:
    """processors.rs:183-192: a no-op hook in the reference."""

    def __init__(self, p: float):
        self.p = float(p)

    def process(self, logits, ctx=None):
        _rows(logits)


class GreedySampler:
    """sampler.rs:9-15: decode::greedy, first maximum wins."""

    def sample(self, logits):
        r, n = _rows(logits)
        out = torch.empty(r, dtype=torch.int32, device=logits.device)
        check(lib.logismos_launch_greedy_argmax(_p(logits), 1, _p(out), r, n, _stream()), "greedy")
        return out


class MultinomialSampler:
    """sampler.rs:17-58. The reference owns an RNG and draws one uniform per call; here a seeded torch
    generator on the device draws one uniform per row, or the caller passes ``uniforms`` explicitly."""

    def __init__(self, seed: int = 0, device="cuda"):
        self.gen = torch.Generator(device=device)
        self.gen.manual_seed(int(seed))

    def sample(self, logits, uniforms=None):
        r, n = _rows(logits)
        if uniforms is None:
            uniforms = torch.rand(r, generator=self.gen, device=logits.device, dtype=torch.float32)
        out = torch.empty(r, dtype=torch.int32, device=logits.device)
        check(lib.logismos_launch_multinomial_f32(_p(logits), r, n, _p(uniforms), _p(out), _stream()), "multinomial")
        return out


class DecodeChain:
    """chain.rs:33-76: processors in insertion order, then the sampler."""

    def __init__(self, sampler):
        self.processors, self.sampler = [], sampler

    def push(self, p):
        self.processors.append(p)
        return self

    def step(self, logits, ctx=None):
        for p in self.processors:
            p.process(logits, ctx)
        return self.sampler.sample(logits)

    def __len__(self):
        return len(self.processors)

    def is_empty(self):
        return not self.processors
