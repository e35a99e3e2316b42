"""The engine at the widths of the 8B shape (hidden 4096, 32 heads over 8 kv heads of 128, feed-forward 14336,
vocabulary 128256) with two layers: the sizes at which the fast kernels really run (tcgen05 products with whole
and cut tiles, the streamed decode product over 148 blocks, TMA attention over many pages), which the tiny
configurations never reach.  Random weights are made once on the device in bfloat16; the 32-bit engine runs the
same values widened.  The oracle is a float64 restatement of the formulas with torch matrix products on the GPU
(src/model.rs:971-1192; the numpy oracle of plain_llama.py would need tens of GB of host memory here); its
rotary frequencies come from plain_llama.rotary_inv_freq.
"""
import math

import numpy as np
import pytest
import torch

import ghost_infer_b200 as gi
from ghost_infer_b200.kernels import ops
import plain_llama as pl
from gpu_helpers import check_logits

pytestmark = pytest.mark.gpu

CFG = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 2, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256,
    "max_position_embeddings": 8192, "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
}
DEV = "cuda:0"


def oracle_logits(w, tokens, places):
    """float64 logits at `places` of one whole sequence."""
    H, KV, hd, eps = 32, 8, 128, CFG["rms_norm_eps"]
    inv = torch.from_numpy(pl.rotary_inv_freq(hd, CFG["rope_theta"], CFG["rope_scaling"])).to(DEV)
    n = len(tokens)
    pos = torch.arange(n, device=DEV, dtype=torch.float32)
    ang = (pos[:, None] * inv[None, :]).double()                    # angles in 32-bit, as the kernels make them
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def norm(x, name):
        return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w[name].double()

    def rope(x, heads):
        x = x.reshape(n, heads, hd)
        a, b = x[..., :hd // 2], x[..., hd // 2:]
        return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)

    x = w["model.embed_tokens.weight"][torch.tensor(tokens, device=DEV)].double()
    causal = torch.ones(n, n, device=DEV, dtype=torch.bool).tril()
    for i in range(CFG["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = norm(x, p + "input_layernorm.weight")
        q = rope(h @ w[p + "self_attn.q_proj.weight"].double().T, H)
        k = rope(h @ w[p + "self_attn.k_proj.weight"].double().T, KV)
        v = (h @ w[p + "self_attn.v_proj.weight"].double().T).reshape(n, KV, hd)
        k, v = k.repeat_interleave(H // KV, dim=1), v.repeat_interleave(H // KV, dim=1)
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(hd)
        s = s.masked_fill(~causal[None], float("-inf"))
        a = torch.einsum("hqk,khd->qhd", torch.softmax(s, dim=-1), v).reshape(n, H * hd)
        x = x + a @ w[p + "self_attn.o_proj.weight"].double().T
        h = norm(x, p + "post_attention_layernorm.weight")
        g, u = h @ w[p + "mlp.gate_proj.weight"].double().T, h @ w[p + "mlp.up_proj.weight"].double().T
        x = x + (g / (1 + torch.exp(-g)) * u) @ w[p + "mlp.down_proj.weight"].double().T
    h = norm(x[places], "model.norm.weight")
    return (h @ w["lm_head.weight"].double().T).cpu().numpy()


@pytest.fixture(scope="module")
def wide():
    model = gi.Model.from_config_dict(CFG)
    gen = torch.Generator(device=DEV)
    gen.manual_seed(7)
    w = {}
    for spec in model.weight_manifest():
        if spec.init == "ones":
            t = 1 + 0.1 * torch.randn(spec.shape, device=DEV, generator=gen)
        else:
            t = 0.02 * torch.randn(spec.shape, device=DEV, generator=gen)
        w[spec.name] = t.to(torch.bfloat16)
    engines = {}

    def engine(dtype):
        if dtype not in engines:
            m = gi.Model.from_config_dict(CFG).bind(w, dtype, DEV)
            engines[dtype] = gi.Engine(m, m.new_cache(max_tokens=64 * 40, max_seq_len=1024, max_slots=8))
        return engines[dtype]

    rng = np.random.default_rng(3)
    tokens = rng.integers(0, CFG["vocab_size"], size=300).tolist()
    places = [0, 1, 63, 64, 127, 128, 200, 267] + list(range(268, 300))
    ref = oracle_logits(w, tokens, places)
    yield engine, tokens, places, ref
    engines.clear()
    w.clear()
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_and_tail_one_by_one(wide, dtype):
    engine, tokens, places, ref = wide
    eng = engine(dtype)
    s = eng.cache.open_slot()
    whole = eng.step([gi.StepEntry(s, tokens, places)]).cpu().numpy()
    eng.cache.close_slot(s)
    check_logits(whole, ref, dtype, f"full width {dtype} whole")
    s = eng.cache.open_slot()
    head = eng.step([gi.StepEntry(s, tokens[:268], places[:8])]).cpu().numpy()
    tail = [eng.step([gi.StepEntry(s, tokens[i:i + 1], [0])]).cpu().numpy()[0] for i in range(268, 300)]
    eng.cache.close_slot(s)
    check_logits(np.concatenate([head, np.stack(tail)]), ref, dtype, f"full width {dtype} tail one by one")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_then_graph_decoding(wide, dtype):
    """The request between two others of other lengths, its tail through the decode runner (CUDA graph, dependent
    launch, deferred partial sums, the L2 request for the next weights)."""
    engine, tokens, places, ref = wide
    eng = engine(dtype)
    rng = np.random.default_rng(4)
    others = [rng.integers(0, CFG["vocab_size"], size=n).tolist() for n in (70, 300)]
    slots = [eng.cache.open_slot() for _ in range(3)]
    was = ops.get_pdl()
    ops.set_pdl(True)
    try:
        out = eng.step([gi.StepEntry(slots[0], others[0], [69]), gi.StepEntry(slots[1], tokens[:268], places[:8]),
                        gi.StepEntry(slots[2], others[1][:268], [])]).cpu().numpy()
        check_logits(out[1:9], ref[:8], dtype, f"full width {dtype} batched prompt")
        eng.cache.close_slot(slots[0])                      # the short one ends earlier
        runner = eng.decoder(slots[1:])
        got = []
        for i in range(268, 300):
            logits = runner.forward(tokens=[tokens[i], others[1][i]])
            got.append(logits[0].cpu().numpy())
        check_logits(np.stack(got), ref[8:], dtype, f"full width {dtype} graph decoding")
        assert ops.gemm_stream_status() == 0 and ops.gemm_tc_status() == 0 and ops.attn_prefill_t5_status() == 0
    finally:
        ops.set_pdl(was)
        for s in slots[1:]:
            eng.cache.close_slot(s)
