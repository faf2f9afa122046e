"""A Llama-shaped decoder, every linear weight-only int8 through torch.compile(backend='hidet_b200'): a prompt pass
and greedy decode steps against the same decoder run eagerly on dequantized weights.

Scaled-down stand-in for the serving configuration of the benchmark specification (32 layers, hidden 4096, FFN 11008,
512-token prompt, 128 decode steps): same structure (RMSNorm, rotary embedding, causal attention over a static
key/value cache, SwiGLU, vocabulary head), small enough to run in seconds.  Both arms see the same tokens (the
eager arm's greedy choices), so a near-tie in one argmax cannot send the two down different paths.
"""
import copy

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import hidet_b200
from hidet_b200 import graph as hg

pytestmark = pytest.mark.gpu

VOCAB, HIDDEN, HEADS, FFN, LAYERS = 512, 256, 4, 688, 3
PROMPT, STEPS = 80, 12          # 80 prompt rows go through the large-M kernel, single rows through the small-M one
CACHE = 96                      # key/value slots per layer (>= PROMPT + STEPS)


class Layer(nn.Module):
    def __init__(self):
        super().__init__()
        self.q = nn.Linear(HIDDEN, HIDDEN, bias=False)
        self.k = nn.Linear(HIDDEN, HIDDEN, bias=False)
        self.v = nn.Linear(HIDDEN, HIDDEN, bias=False)
        self.o = nn.Linear(HIDDEN, HIDDEN, bias=False)
        self.gate = nn.Linear(HIDDEN, FFN, bias=False)
        self.up = nn.Linear(HIDDEN, FFN, bias=False)
        self.down = nn.Linear(FFN, HIDDEN, bias=False)
        self.n1 = nn.Parameter(torch.ones(HIDDEN))
        self.n2 = nn.Parameter(torch.ones(HIDDEN))


def rms(x, w):
    return (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5)).to(x.dtype) * w


def rope(x, cos, sin):
    # x [1, H, T, D]; cos, sin [T, D / 2]
    x1, x2 = x[..., 0::2], x[..., 1::2]
    out = torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1)
    return out.flatten(-2).to(x.dtype)


class Decoder(nn.Module):
    def __init__(self):
        super().__init__()
        self.embed = nn.Embedding(VOCAB, HIDDEN)
        self.layers = nn.ModuleList(Layer() for _ in range(LAYERS))
        self.norm = nn.Parameter(torch.ones(HIDDEN))
        self.head = nn.Linear(HIDDEN, VOCAB, bias=False)
        d = HIDDEN // HEADS
        freq = 1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d))
        angle = torch.arange(CACHE).float()[:, None] * freq[None, :]
        self.register_buffer('cos', angle.cos())
        self.register_buffer('sin', angle.sin())
        for p in self.parameters():
            if p.dim() == 2:
                nn.init.normal_(p, std=0.02)

    def forward(self, ids, k_cache, v_cache, pos):
        """ids [1, T]; caches [LAYERS, 1, HEADS, CACHE, D]; pos [T], the cache slots of these tokens.
        Returns the last token's logits and the caches with these tokens' keys and values added."""
        t = ids.shape[1]
        d = HIDDEN // HEADS
        x = self.embed(ids)
        cos = self.cos.index_select(0, pos).to(x.dtype)
        sin = self.sin.index_select(0, pos).to(x.dtype)
        slots = torch.arange(CACHE, device=ids.device)
        mask = slots[None, :] <= pos[:, None]            # query at slot p sees keys in slots <= p
        keys, values = [], []
        for i, layer in enumerate(self.layers):
            y = rms(x, layer.n1)
            q = layer.q(y).view(1, t, HEADS, d).transpose(1, 2)
            k = layer.k(y).view(1, t, HEADS, d).transpose(1, 2)
            v = layer.v(y).view(1, t, HEADS, d).transpose(1, 2)
            q, k = rope(q, cos, sin), rope(k, cos, sin)
            kc = k_cache[i].index_copy(2, pos, k)
            vc = v_cache[i].index_copy(2, pos, v)
            a = F.scaled_dot_product_attention(q, kc, vc, attn_mask=mask)
            x = x + layer.o(a.transpose(1, 2).reshape(1, t, HIDDEN))
            y = rms(x, layer.n2)
            x = x + layer.down(F.silu(layer.gate(y)) * layer.up(y))
            keys.append(kc)
            values.append(vc)
        logits = self.head(rms(x, self.norm)[:, -1])
        return logits, torch.stack(keys), torch.stack(values)


def empty_caches(device, dtype):
    shape = (LAYERS, 1, HEADS, CACHE, HIDDEN // HEADS)
    return torch.zeros(shape, device=device, dtype=dtype), torch.zeros(shape, device=device, dtype=dtype)


def with_dequantized_weights(model):
    """The eager arm: every linear's weight replaced by dequantize(quantize(W)) per output channel."""
    ref = copy.deepcopy(model)
    for mod in ref.modules():
        if isinstance(mod, nn.Linear):
            w_kn = mod.weight.detach().t().contiguous()
            wq, scale = hidet_b200.symmetric_quantize(w_kn, 'int8', dims=0)
            mod.weight.data.copy_(hidet_b200.symmetric_dequantize(wq, scale, dims=0).t())
    return ref


def run(model, prompt, forced=None):
    """Prompt pass, then STEPS single-token passes.  Feeds its own greedy tokens, or `forced` ones."""
    device = prompt.device
    kc, vc = empty_caches(device, torch.float16)
    logits, kc, vc = model(prompt, kc, vc, torch.arange(PROMPT, device=device))
    all_logits, tokens = [logits], []
    for step in range(STEPS):
        nxt = forced[step] if forced is not None else logits.argmax(-1)
        tokens.append(nxt)
        logits, kc, vc = model(nxt.view(1, 1), kc, vc, torch.full((1,), PROMPT + step, device=device, dtype=torch.long))
        all_logits.append(logits)
    return torch.cat(all_logits).float(), tokens


def test_compiled_int8_decoder_follows_the_eager_decoder_on_dequantized_weights():
    hg.register()
    torch.manual_seed(7)
    model = Decoder().half().cuda().eval()
    prompt = torch.randint(0, VOCAB, (1, PROMPT), device='cuda')
    with torch.no_grad():
        ref_logits, ref_tokens = run(with_dequantized_weights(model), prompt)
        compiled = torch.compile(model, backend='hidet_b200', options={'precision': 'int8'}, dynamic=False)
        got_logits, _ = run(compiled, prompt, forced=ref_tokens)
        again_logits, _ = run(compiled, prompt, forced=ref_tokens)
        plain_logits, _ = run(model, prompt, forced=ref_tokens)
    assert torch.equal(got_logits, again_logits)
    assert torch.isfinite(got_logits).all()
    scale = ref_logits.abs().max()
    # same weights in both arms (int8 codes x scales); what differs is where sums are rounded
    assert (got_logits - ref_logits).abs().max() <= 1e-2 * scale
    agree = (got_logits.argmax(-1) == ref_logits.argmax(-1)).float().mean()
    assert agree >= 0.9
    # and the compiled arm did run on quantized weights: it is closer to the dequantized-weight decoder
    # than the unquantized decoder is
    assert (plain_logits - ref_logits).abs().max() > (got_logits - ref_logits).abs().max()
    assert hidet_b200.ffi.func('b200q_check_status')() == hidet_b200.ffi.OK
