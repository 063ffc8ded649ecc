"""Runs one kernel of hi_b200 alone on a small, fixed case, for `ncu -k regex:<kernel>`, or a
whole step of a few layers without CUDA graphs, for a list of its launches.

    python -m hi_b200.kernels.cases decode_attention [batch] [context]
    python -m hi_b200.kernels.cases expert_gemv [batch]
    python -m hi_b200.kernels.cases expert_tc [tokens] [experts]
    python -m hi_b200.kernels.cases prefill_attention [tokens]
    python -m hi_b200.kernels.cases decode_step [batch] [context] [layers]
    python -m hi_b200.kernels.cases prefill_step [tokens] [layers]

Sizes are the Scout layer's (40 heads, 8 kv heads, head_dim 128; hidden 5120, 16 experts of
intermediate 8192); inputs are larger than L2 and well under a few GB.
"""
import sys

import torch

from . import ops

DEV = "cuda:0"


def decode_attention(batch=8, context=8192, page=64):
    nh, nkv, hd = 40, 8, 128
    blocks = -(-context // page)
    g = torch.Generator(device=DEV).manual_seed(0)
    kp = torch.randn(batch * blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    vp = torch.randn(batch * blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    bt = torch.randperm(batch * blocks, device=DEV, generator=g).to(torch.int32).view(batch, blocks).contiguous()
    q = torch.randn(batch, nh, hd, device=DEV, generator=g).to(torch.bfloat16)
    pos = torch.full((batch,), context - 1, dtype=torch.int32, device=DEV)
    sot = torch.arange(batch, dtype=torch.int32, device=DEV)
    for _ in range(3):
        out = ops.decode_attention(q, kp, vp, bt, sot, pos, 0, 0, hd ** -0.5, context)
    torch.cuda.synchronize()
    return out


def expert_gemv(batch=8):
    hidden, experts, inter = 5120, 16, 8192
    g = torch.Generator(device=DEV).manual_seed(0)
    x = torch.randn(batch, hidden, device=DEV, generator=g).to(torch.bfloat16)
    wg = (torch.randn(experts, inter, hidden, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    wu = (torch.randn(experts, inter, hidden, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    wd = (torch.randn(experts, hidden, inter, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    ids = torch.randint(0, experts, (batch, 1), device=DEV, generator=g).to(torch.int32)
    scores = torch.rand(batch, 1, device=DEV, generator=g)
    plan = ops.moe_plan(ids, experts)
    for _ in range(3):
        act = ops.moe_gate_up(x, plan, 1, wg, wu, scores, True)
        y = ops.moe_down(act, wd, plan, True)
    torch.cuda.synchronize()
    return y


def expert_tc(tokens=1024, experts=8):
    """The tcgen05 grouped products at prefill shape: about 128 rows per expert."""
    hidden, inter = 5120, 8192
    g = torch.Generator(device=DEV).manual_seed(0)
    x = torch.randn(tokens, hidden, device=DEV, generator=g).to(torch.bfloat16)
    wg = (torch.randn(experts, inter, hidden, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    wu = (torch.randn(experts, inter, hidden, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    wd = (torch.randn(experts, hidden, inter, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    ids = torch.randint(0, experts, (tokens, 1), device=DEV, generator=g).to(torch.int32)
    scores = torch.rand(tokens, 1, device=DEV, generator=g)
    plan = ops.moe_plan(ids, experts)
    for _ in range(3):
        act = ops.moe_gate_up_tc(x, plan, 1, wg, wu, scores)
        y = ops.moe_down_tc(act, wd, plan)
    ops.check_tc_status()
    return y


def prefill_attention(tokens=2048, page=64):
    nh, nkv, hd = 40, 8, 128
    blocks = -(-tokens // page)
    g = torch.Generator(device=DEV).manual_seed(0)
    kp = torch.randn(blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    vp = torch.randn(blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    bt = torch.randperm(blocks, device=DEV, generator=g).to(torch.int32).view(1, blocks).contiguous()
    q = torch.randn(tokens, nh, hd, device=DEV, generator=g).to(torch.bfloat16)
    pos = torch.arange(tokens, dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, tokens], dtype=torch.int32, device=DEV)
    for _ in range(3):
        out = ops.prefill_attention(q, kp, vp, bt, cu, pos, 1, tokens, 0, 0, hd ** -0.5)
        out = ops.prefill_attention_tc(q, kp, vp, bt, cu, pos, 1, tokens, 0, 0, hd ** -0.5)
    ops.check_tc_status()
    return out


SCOUT_LAYER = {
    "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
    "vocab_size": 202048, "hidden_size": 5120, "num_attention_heads": 40, "num_key_value_heads": 8, "head_dim": 128,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 1.0,
                     "original_max_position_embeddings": 8192},
    "attention_chunk_size": 8192, "nope_layer_interval": 4, "use_qk_norm": True,
    "attn_temperature_tuning": True, "floor_scale": 8192, "attn_scale": 0.1,
    "interleave_moe_layer_step": 1, "num_local_experts": 16, "num_experts_per_tok": 1,
    "intermediate_size": 8192, "intermediate_size_mlp": 16384, "tie_word_embeddings": False,
    "max_position_embeddings": 262144,
}


def _engine(layers, tokens, slots):
    from ..engine.core import Engine

    return Engine.from_config(dict(SCOUT_LAYER, num_hidden_layers=layers), seed=0, dtype="bfloat16", device=DEV,
                              kv_page_size=64, kv_cache_tokens=tokens, max_active_requests=slots, use_cuda_graphs=False)


def decode_step(batch=8, context=8192, layers=2):
    """Three decode steps of `batch` requests at `context` cached tokens, every kernel launched on its own."""
    from ..engine.core import StepEntry

    eng = _engine(layers, batch * (context + 128), batch + 1)
    for i in range(batch):
        eng.assume_cached(i, context - 8)
    g = torch.Generator().manual_seed(0)
    for _ in range(3):
        eng.step([StepEntry(i, [int(torch.randint(0, 202048, (1,), generator=g))], [0]) for i in range(batch)])
    torch.cuda.synchronize()


def prefill_step(tokens=2048, layers=2):
    """Three prompts of `tokens` tokens, each in one step."""
    from ..engine.core import StepEntry

    eng = _engine(layers, tokens + 128, 2)
    g = torch.Generator().manual_seed(0)
    for i in range(3):
        eng.step([StepEntry(i, torch.randint(0, 202048, (tokens,), generator=g).tolist(), [tokens - 1])])
        eng.finish(i)
    torch.cuda.synchronize()


if __name__ == "__main__":
    what = sys.argv[1]
    args = [int(a) for a in sys.argv[2:]]
    {"decode_attention": decode_attention, "expert_gemv": expert_gemv, "expert_tc": expert_tc,
     "prefill_attention": prefill_attention, "decode_step": decode_step, "prefill_step": prefill_step}[what](*args)
    print("ok")
