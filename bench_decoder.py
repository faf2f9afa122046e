"""A Llama-shaped decoder with every linear weight-only int8, compiled through torch.compile(backend='hidet_b200').

This is the serving configuration of the benchmark specification: a Llama-2-7B-shaped decoder (32 layers, hidden
4096, 32 heads, FFN 11008 SwiGLU, RMSNorm, rotary embedding, vocabulary 32000) with random-init fp16 weights, batch
1, a 512-token prompt and 128 greedy decode steps.  The reference's flow for it is
torch.compile(model, backend='hidet') with its quantization pass
(python/hidet/graph/frontend/torch/dynamo_backends.py:78-92,144-175); there is no checkpoint or dataset here, so
weights and token ids are seeded random numbers of the same shapes.

The model keeps a static key/value cache and is called in two shapes only (the prompt pass and the one-token
step), so there is one compiled graph per shape and the step is replayed as a CUDA graph (hidet_b200.CudaGraph).
`run_config` returns prompt time, time per decode step and the parity of the compiled int8 model's logits with the
same decoder run eagerly in fp32 on dequantized weights (teacher-forced with that arm's tokens).

Used by bench.py (`--config4`, and as the `config4` block of the default line) and by tests/test_decoder_gpu.py.
"""
from __future__ import annotations

import copy
import time
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class DecoderConfig:
    vocab: int = 32000
    hidden: int = 4096
    heads: int = 32
    ffn: int = 11008
    layers: int = 32
    prompt: int = 512
    steps: int = 128

    @property
    def cache(self) -> int:
        return -(-(self.prompt + self.steps) // 64) * 64


LLAMA_7B = DecoderConfig()
SMALL = DecoderConfig(vocab=512, hidden=256, heads=4, ffn=688, layers=3, prompt=80, steps=12)


class Layer(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        h, f = cfg.hidden, cfg.ffn
        self.q = nn.Linear(h, h, bias=False)
        self.k = nn.Linear(h, h, bias=False)
        self.v = nn.Linear(h, h, bias=False)
        self.o = nn.Linear(h, h, bias=False)
        self.gate = nn.Linear(h, f, bias=False)
        self.up = nn.Linear(h, f, bias=False)
        self.down = nn.Linear(f, h, bias=False)
        self.n1 = nn.Parameter(torch.ones(h))
        self.n2 = nn.Parameter(torch.ones(h))


def rms(x, w):
    return (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5)).to(x.dtype) * w


def rope(x, cos, sin):
    # x [1, H, T, D]; cos, sin [T, D / 2]
    x1, x2 = x[..., 0::2], x[..., 1::2]
    out = torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1)
    return out.flatten(-2).to(x.dtype)


class Decoder(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab, cfg.hidden)
        self.layers = nn.ModuleList(Layer(cfg) for _ in range(cfg.layers))
        self.norm = nn.Parameter(torch.ones(cfg.hidden))
        self.head = nn.Linear(cfg.hidden, cfg.vocab, bias=False)
        d = cfg.hidden // cfg.heads
        freq = 1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d))
        angle = torch.arange(cfg.cache).float()[:, None] * freq[None, :]
        self.register_buffer('cos', angle.cos())
        self.register_buffer('sin', angle.sin())
        for p in self.parameters():
            if p.dim() == 2:
                nn.init.normal_(p, std=0.02)

    def forward(self, ids, k_cache, v_cache, pos):
        """ids [1, T]; caches [layers, 1, heads, cache, D], updated in place; pos [T], the cache slots of these
        tokens.  Returns the last token's logits."""
        cfg = self.cfg
        t = ids.shape[1]
        d = cfg.hidden // cfg.heads
        x = self.embed(ids)
        cos = self.cos.index_select(0, pos).to(x.dtype)
        sin = self.sin.index_select(0, pos).to(x.dtype)
        slots = torch.arange(cfg.cache, device=ids.device)
        mask = slots[None, :] <= pos[:, None]            # query at slot p sees keys in slots <= p
        for i, layer in enumerate(self.layers):
            y = rms(x, layer.n1)
            q = layer.q(y).view(1, t, cfg.heads, d).transpose(1, 2)
            k = layer.k(y).view(1, t, cfg.heads, d).transpose(1, 2)
            v = layer.v(y).view(1, t, cfg.heads, d).transpose(1, 2)
            q, k = rope(q, cos, sin), rope(k, cos, sin)
            k_cache[i].index_copy_(2, pos, k)
            v_cache[i].index_copy_(2, pos, v)
            a = F.scaled_dot_product_attention(q, k_cache[i], v_cache[i], attn_mask=mask)
            x = x + layer.o(a.transpose(1, 2).reshape(1, t, cfg.hidden))
            y = rms(x, layer.n2)
            x = x + layer.down(F.silu(layer.gate(y)) * layer.up(y))
        return self.head(rms(x, self.norm)[:, -1])


def empty_caches(cfg: DecoderConfig, device, dtype=torch.float16):
    shape = (cfg.layers, 1, cfg.heads, cfg.cache, cfg.hidden // cfg.heads)
    return torch.zeros(shape, device=device, dtype=dtype), torch.zeros(shape, device=device, dtype=dtype)


def with_dequantized_weights(model: Decoder) -> Decoder:
    """The eager arm: every linear's weight replaced by dequantize(quantize(W)) per output channel, and the
    embedding table by dequantize(quantize(table)) per row, as the rewrite rules quantize them."""
    import hidet_b200

    ref = copy.deepcopy(model)
    for mod in ref.modules():
        if isinstance(mod, nn.Linear):
            w_kn = mod.weight.detach().t().contiguous()
            wq, scale = hidet_b200.symmetric_quantize(w_kn, 'int8', dims=0)
            mod.weight.data.copy_(hidet_b200.symmetric_dequantize(wq, scale, dims=0).t())
        elif isinstance(mod, nn.Embedding):
            wq, scale = hidet_b200.symmetric_quantize(mod.weight.detach(), 'int8', dims=-1)
            mod.weight.data.copy_(hidet_b200.symmetric_dequantize(wq, scale, dims=-1))
    return ref


def greedy(model, cfg: DecoderConfig, prompt, steps: int, forced=None, dtype=torch.float16):
    """Prompt pass, then `steps` one-token passes, eagerly (no CUDA graph).  Feeds its own greedy tokens, or
    `forced` ones.  Returns (logits of every pass [steps + 1, vocab], tokens)."""
    device = prompt.device
    kc, vc = empty_caches(cfg, device, dtype)
    logits = model(prompt, kc, vc, torch.arange(cfg.prompt, device=device))
    all_logits, tokens = [logits], []
    for step in range(steps):
        nxt = forced[step] if forced is not None else logits.argmax(-1)
        tokens.append(nxt)
        logits = model(nxt.view(1, 1), kc, vc, torch.full((1,), cfg.prompt + step, device=device, dtype=torch.long))
        all_logits.append(logits)
    return torch.cat(all_logits).float(), tokens


def run_config(cfg: DecoderConfig = LLAMA_7B, parity_steps: int = 8, seed: int = 7) -> dict:
    """Builds the decoder, compiles it with int8 linears, times the prompt pass and the decode steps (the step
    replayed as one CUDA graph) and checks the logits of the first `parity_steps` passes against the eager
    decoder on dequantized weights."""
    import hidet_b200
    from hidet_b200 import graph as hg

    hg.register()
    device = torch.device('cuda', torch.cuda.current_device())
    torch.manual_seed(seed)
    with torch.device(device):
        model = Decoder(cfg).half().eval()
    prompt = torch.randint(0, cfg.vocab, (1, cfg.prompt), device=device, generator=torch.Generator(device=device).manual_seed(seed))
    out = {'model': {'layers': cfg.layers, 'hidden': cfg.hidden, 'heads': cfg.heads, 'ffn': cfg.ffn, 'vocab': cfg.vocab},
           'prompt_tokens': cfg.prompt, 'decode_steps': cfg.steps, 'batch': 1}
    with torch.no_grad():
        # ---- parity: all arms see the tokens the fp32 arm chooses greedily ----
        # The oracle is the same decoder on dequantized weights in fp32 (no rounding between layers); beside it,
        # the error of the eager fp16 decoder on the same weights shows what fp16 rounding alone costs.
        ref16 = with_dequantized_weights(model)
        ref32 = copy.deepcopy(ref16).float()
        ref_logits, ref_tokens = greedy(ref32, cfg, prompt, parity_steps, dtype=torch.float32)
        del ref32
        eager_logits, _ = greedy(ref16, cfg, prompt, parity_steps, forced=ref_tokens)
        del ref16
        torch.cuda.empty_cache()
        t0 = time.perf_counter()
        compiled = torch.compile(model, backend='hidet_b200', options={'precision': 'int8'}, dynamic=False)
        got_logits, _ = greedy(compiled, cfg, prompt, parity_steps, forced=ref_tokens)
        torch.cuda.synchronize()
        out['compile_and_first_passes_s'] = round(time.perf_counter() - t0, 1)
        top = ref_logits.abs().max().item()
        out['parity'] = {'against': 'the decoder on dequantized weights in fp32, teacher-forced', 'passes_compared': parity_steps + 1,
                         'max_abs_err_over_max_ref': (got_logits - ref_logits).abs().max().item() / top,
                         'eager_f16_max_abs_err_over_max_ref': (eager_logits - ref_logits).abs().max().item() / top,
                         'argmax_agreement': (got_logits.argmax(-1) == ref_logits.argmax(-1)).float().mean().item()}

        # ---- timing ----
        kc, vc = empty_caches(cfg, device)
        positions = torch.arange(cfg.prompt, device=device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        prompt_ms = []
        for _ in range(3):
            torch.cuda.synchronize()
            e0.record()
            logits = compiled(prompt, kc, vc, positions)
            e1.record()
            torch.cuda.synchronize()
            prompt_ms.append(e0.elapsed_time(e1))
        out['prompt_ms'] = round(min(prompt_ms), 3)
        out['prompt_tokens_per_s'] = round(cfg.prompt / (min(prompt_ms) * 1e-3), 1)

        ids_static = logits.argmax(-1).view(1, 1).clone()
        pos_static = torch.full((1,), cfg.prompt, device=device, dtype=torch.long)
        step_graph = hidet_b200.CudaGraph(lambda: [ids_static, pos_static], lambda inp: [compiled(inp[0], kc, vc, inp[1])], ref_objs=[compiled, kc, vc])
        stream = torch.cuda.current_stream()
        generated = []
        torch.cuda.synchronize()
        e0.record()
        for step in range(cfg.steps):
            pos_static.fill_(cfg.prompt + step)
            (step_logits,) = step_graph.run_async()
            ids_static.copy_(step_logits.argmax(-1).view(1, 1))
            generated.append(ids_static.clone())
        e1.record()
        stream.synchronize()
        decode_ms = e0.elapsed_time(e1)
        out['ms_per_decode_step'] = round(decode_ms / cfg.steps, 4)
        out['decode_tokens_per_s'] = round(cfg.steps / (decode_ms * 1e-3), 1)
        out['generated_tokens'] = int(torch.cat(generated).numel())
        weight_bytes = sum(m.weight.numel() for m in model.modules() if isinstance(m, nn.Linear))
        out['int8_weight_bytes_per_step'] = weight_bytes
        out['weight_stream_GBps'] = round(weight_bytes / (decode_ms / cfg.steps * 1e-3) / 1e9, 1)
        out['kernel_time_of_a_step'] = kernel_time_of_a_step(step_graph)
        assert hidet_b200.ffi.func('b200q_check_status')() == hidet_b200.ffi.OK
    return out


def kernel_time_of_a_step(step_graph, replays: int = 3):
    """Device time of the kernels of one decode step by kind, from torch.profiler's kernel records of a few replays of
    the step's CUDA graph: how much of the step is the quantized-linear path and how much the rest of the decoder
    (attention, normalisation, rotary embedding and the other element-wise kernels torch launches).  None when the
    profiler gives no kernel records."""
    try:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(replays):
                step_graph.run_async()
            torch.cuda.synchronize()
        kinds = {'qlinear': 0.0, 'embedding_dequant': 0.0, 'other': 0.0}
        launches = {'qlinear': 0, 'embedding_dequant': 0, 'other': 0}
        for row in prof.key_averages():
            t = float(getattr(row, 'device_time_total', 0.0) or getattr(row, 'cuda_time_total', 0.0) or 0.0)
            if t <= 0.0:
                continue
            kind = 'qlinear' if 'qlinear' in row.key else 'embedding_dequant' if 'embedding_dequant' in row.key else 'other'
            kinds[kind] += t
            launches[kind] += int(row.count)
        total = sum(kinds.values())
        if total <= 0.0:
            return None
        return {'us_per_step': {k: round(v / replays, 1) for k, v in kinds.items()},
                'launches_per_step': {k: v // replays for k, v in launches.items()},
                'share_of_kernel_time_in_the_quantized_path': round((kinds['qlinear'] + kinds['embedding_dequant']) / total, 4)}
    except Exception as e:  # the profiler is optional equipment
        return {'unavailable': '{}: {}'.format(type(e).__name__, e)}


if __name__ == '__main__':
    import json
    import sys

    print(json.dumps(run_config(SMALL if '--small' in sys.argv else LLAMA_7B)))
