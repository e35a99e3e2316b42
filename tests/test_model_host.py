"""What a model decides on the host, checked without a GPU: the context it allows, the names its parts give their
tensors, and what a step's context offers to parts."""
import warnings

import pytest
import torch

import ghost_infer_b200 as gi
from ghost_infer_b200.engine.step import StepContext
from ghost_infer_b200.parts import PartSpec, lookup
from ghost_infer_b200.weights.random_init import random_tensors
from conftest import TINY_A


def bound_on_cpu(raw):
    model = gi.Model.from_config_dict(raw)
    return model.bind(random_tensors(model.weight_manifest(), 0, torch.float32), "float32", device="cpu")


def test_the_context_is_never_longer_than_the_model_s_positions_unless_asked():
    """The reference clamps a session's context to the model's (`ctx.min(max_ctx)`, src/model.rs:732)."""
    model = bound_on_cpu(TINY_A)                                    # max_position_embeddings 128
    assert model.new_cache(max_tokens=64 * 8).max_seq_len == 128
    assert model.new_cache(max_tokens=64 * 8, max_seq_len=100).max_seq_len == 100
    with pytest.warns(UserWarning, match="128 positions"):
        assert model.new_cache(max_tokens=64 * 8, max_seq_len=300).max_seq_len == 128
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        assert model.new_cache(max_tokens=64 * 8, max_seq_len=300, beyond_trained_positions=True).max_seq_len == 300
    # the pool bounds it too: a sequence that keeps every position cannot hold more than all pages
    assert model.new_cache(max_tokens=64, max_seq_len=128).max_seq_len == 64


def test_parts_name_their_tensors_through_the_specification():
    att = lookup("mixer", "gqa_attention")
    base = {"hidden_size": 8, "num_heads": 2, "num_kv_heads": 1, "head_dim": 4, "scale": 0.5, "window": None, "position": None}
    assert [w.name for w in att(base, "L.").weights()] == [f"L.self_attn.{k}_proj.weight" for k in "qkvo"]
    renamed = att(dict(base, tensor_names={"q": "wq", "o": "attn_out.w"}), "L.")
    assert [w.name for w in renamed.weights()] == ["L.wq", "L.self_attn.k_proj.weight", "L.self_attn.v_proj.weight", "L.attn_out.w"]
    ffn = lookup("feed_forward", "swiglu")({"hidden_size": 8, "intermediate_size": 16, "tensor_names": {"gate": "w1", "up": "w3", "down": "w2"}}, "F.")
    assert [w.name for w in ffn.weights()] == ["F.w1", "F.w3", "F.w2"]
    norm = lookup("norm", "rmsnorm")({"size": 8, "eps": 1e-5, "tensor_names": {"weight": "scale"}}, "N.")
    assert [w.name for w in norm.weights()] == ["N.scale"]


def test_a_recorded_step_refuses_host_side_lists_in_words():
    ctx = StepContext()
    assert ctx.host_slots == [] and ctx.host_q_lens == [] and ctx.host_pos0 == []
    ctx._host_slots = ctx._host_q_lens = ctx._host_pos0 = None      # what a recorded step carries
    for name in ("host_slots", "host_q_lens", "host_pos0"):
        with pytest.raises(RuntimeError, match="plans_on_host"):
            getattr(ctx, name)


def test_a_step_asks_the_mixer_for_its_plan_unless_one_was_recorded():
    class M:
        def decode_plan(self, n_seqs, max_kv_len, sm_count, kv_lens=None):
            return ("plan", n_seqs, max_kv_len, sm_count)

    m, ctx = M(), StepContext()
    ctx.n_seqs, ctx.max_kv_len, ctx.sm_count, ctx.is_decode = 3, 500, 10, True
    assert ctx.plan_of(m) == ("plan", 3, 500, 10)
    ctx.fixed_plans = {id(m): "recorded"}
    assert ctx.plan_of(m) == "recorded"
    ctx.fixed_plans, ctx.is_decode = None, False
    assert ctx.plan_of(m) is None                                   # a prompt step has no decode plan


def test_a_wait_that_ran_out_inside_a_kernel_is_never_silent(monkeypatch):
    """The tensor-core kernels bound every wait and record which one ran out; the entry points read the records before
    they hand anything back (`ops.check_status`)."""
    from ghost_infer_b200.kernels import ops
    from ghost_infer_b200.kernels.library import KernelError
    codes = {"gemm_tc_status": 0, "gemm_stream_status": 0, "attn_prefill_t5_status": 0}
    for name in codes:
        monkeypatch.setattr(ops, name, lambda name=name: codes[name])
    ops.check_status()                                              # nothing recorded: nothing said
    codes["attn_prefill_t5_status"] = 2
    with pytest.raises(KernelError, match="prompt attention \\(wait 2\\)"):
        ops.check_status()
    codes["gemm_stream_status"] = 3
    with pytest.raises(KernelError, match="decode product \\(wait 3\\), prompt attention"):
        ops.check_status()
