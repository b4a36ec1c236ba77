"""Shared by the tests: the tiny configurations, request sets, tolerances, trace replay driver."""
import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Two tiny Llama configurations that differ in every size and option, a third with awkward
# sizes (width 68 is no multiple of 8, vocabulary 307 is prime, 100 is no multiple of 8), and two
# narrow ones with the head geometry of the sizes the benchmark is quoted on, so that whole models
# run through the tensor-core kernels: D has head size 64 in groups of 4 (the 1B geometry, tied,
# llama3 factor 32), E head size 128 with an untied head (the 3B / 8B geometry).
TINY = {
    "A": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=64,
                    intermediate_size=192, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=16, vocab_size=256, rope_theta=10000.0,
                    rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=128),
        seed=0, std=0.02, norm_mean=1.0, norm_std=0.0),
    "B": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=96,
                    intermediate_size=256, num_hidden_layers=3, num_attention_heads=3,
                    num_key_value_heads=1, head_dim=32, vocab_size=512, rope_theta=500000.0,
                    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0,
                                      high_freq_factor=4.0, original_max_position_embeddings=64),
                    rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=256),
        seed=7, std=0.05, norm_mean=1.0, norm_std=0.1),
    "C": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=68,
                    intermediate_size=100, num_hidden_layers=1, num_attention_heads=6,
                    num_key_value_heads=3, head_dim=48, vocab_size=307, rope_theta=1000.0,
                    rope_scaling=dict(rope_type="linear", factor=2.0),
                    rms_norm_eps=1e-4, tie_word_embeddings=False, max_position_embeddings=512),
        seed=3, std=0.08, norm_mean=1.0, norm_std=0.2),
    "D": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=512,
                    intermediate_size=1536, num_hidden_layers=2, num_attention_heads=8,
                    num_key_value_heads=2, head_dim=64, vocab_size=2048, rope_theta=500000.0,
                    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0,
                                      high_freq_factor=4.0, original_max_position_embeddings=8192),
                    rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=1024),
        seed=11, std=0.04, norm_mean=1.0, norm_std=0.05),
    "E": dict(
        config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=384,
                    intermediate_size=1024, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=128, vocab_size=1000, rope_theta=500000.0,
                    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0,
                                      high_freq_factor=4.0, original_max_position_embeddings=8192),
                    rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=1024),
        seed=13, std=0.05, norm_mean=1.0, norm_std=0.05),
}


def make_model_dir(path, name, dtype=torch.bfloat16):
    from llama_rs_metal_b200.engine.session import write_random_model
    spec = TINY[name]
    return write_random_model(path, spec["config"], seed=spec["seed"], std=spec["std"],
                              norm_mean=spec["norm_mean"], norm_std=spec["norm_std"], dtype=dtype)


# Tiny Kikalix configurations. K1: odd sizes throughout (no size a multiple of 16, key, value and
# query head counts all different, a layer without a feed-forward, a loop that starts after the
# first layer and runs three times, windows shorter and longer than a page, one and three chosen
# experts, a rotation of part of the head). K2: head size 64 on both sides of the parallel mixer,
# so that bfloat16 runs the tensor-core products and the tiled attention kernels with the distance
# penalty; its loop starts at the first layer. K3: a window of exactly one page, a convolution of
# one tap (no tail), no loop, no feed-forward.
def _moe(ff, limit, experts, top):
    return dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, top=top))


KIKALIX = {
    "K1": dict(
        config=dict(architecture="Kikalix", vocab=211, width=72, norm=dict(eps=1e-6), layers=[
            dict(type="parallel", mixer=dict(
                left=dict(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, mask=dict(size=7)), left_scale=0.7,
                right=dict(heads=4, kv_heads=2, dim=24, vdim=8, conv=3, decay_rank=5, gate_rank=7), right_scale=1.3),
                mlp=_moe(40, 1.0, 5, 3)),
            dict(type="retention", mixer=dict(heads=3, dim=20, vdim=12, decay=[0.9, 0.97, 0.995],
                                              rot=dict(dims=8, base=100.0)), mlp=None),
            dict(type="parallel", mixer=dict(
                left=dict(heads=2, kv_heads=2, dim=8, vdim=8, scale=0.5, mask=dict(size=70)), left_scale=1.0,
                right=dict(heads=2, kv_heads=1, dim=16, vdim=16, conv=2, decay_rank=3, gate_rank=3), right_scale=0.25),
                mlp=_moe(24, 0.5, 3, 1)),
        ], loop=dict(start=1, stop=3, times=3)), seed=21, std=0.12),
    "K2": dict(
        config=dict(architecture="Kikalix", vocab=512, width=320, norm=dict(eps=2e-5), layers=[
            dict(type="retention", mixer=dict(heads=4, dim=64, vdim=64, decay=[0.98, 0.99, 0.995, 0.999],
                                              rot=dict(dims=64, base=10000.0)), mlp=_moe(128, 2.0, 4, 2)),
            dict(type="parallel", mixer=dict(
                left=dict(heads=8, kv_heads=2, dim=64, vdim=64, scale=0.125, mask=dict(size=100)), left_scale=0.5,
                right=dict(heads=4, kv_heads=4, dim=64, vdim=64, conv=4, decay_rank=16, gate_rank=16), right_scale=0.5),
                mlp=_moe(128, 2.0, 4, 2)),
        ], loop=dict(start=0, stop=1, times=2)), seed=22, std=0.06),
    "K3": dict(
        config=dict(architecture="Kikalix", vocab=300, width=64, norm=dict(eps=1e-5), layers=[
            dict(type="parallel", mixer=dict(
                left=dict(heads=2, kv_heads=1, dim=32, vdim=32, scale=0.2, mask=dict(size=64)), left_scale=1.0,
                right=dict(heads=1, kv_heads=1, dim=8, vdim=8, conv=1, decay_rank=2, gate_rank=2), right_scale=1.0),
                mlp=None),
            dict(type="retention", mixer=dict(heads=1, dim=16, vdim=48, decay=[0.9375], rot=dict(dims=16, base=50.0)),
                 mlp=None),
        ]), seed=23, std=0.15),
}


def make_kikalix_dir(path, name, dtype=torch.bfloat16, steady_routing=False):
    """A model folder of a tiny Kikalix configuration with seeded random weights. Norm weights,
    biases and the other vectors are N(0, 0.2); the routers' matrices are eight times larger than
    the rest, so that the experts' weights differ from token to token. The choice of experts is a
    step function of the router's input: with random weights a runner-up now and then comes
    within a rounding of bfloat16 activations of the last chosen expert, and the engine and the
    float64 implementation then choose differently. `steady_routing` is for comparisons in
    bfloat16: the routers' matrices keep their size and their biases are 0, 6, 12, ..., so the same
    experts win for every token (their weights still depend on the token) and no comparison
    rests on a close call."""
    from llama_rs_metal_b200.engine.model import DecoderModel
    from llama_rs_metal_b200.registry import find_architecture
    from llama_rs_metal_b200.runtime import Runtime
    from llama_rs_metal_b200.weights.random_init import random_tensors, write_model_folder
    spec = KIKALIX[name] if isinstance(name, str) else name   # or a spec of the caller's own
    arch = find_architecture(spec["config"])
    config = arch.config_class.from_dict(spec["config"])
    model = DecoderModel(arch.plan(config), Runtime(torch.device("cpu"), torch.float32))
    tensors = random_tensors(model.tensor_specs(), spec["seed"], std=spec["std"], vector_mean=0.0, vector_std=0.2,
                             dtype=dtype)
    for name_, t in tensors.items():
        if name_.endswith(".router") and not steady_routing:
            t.mul_(8.0)
        if name_.endswith(".router.b") and steady_routing:
            t.copy_(6.0 * torch.arange(t.numel()))
    return write_model_folder(path, config.to_dict(), tensors, spec["seed"])


# Tiny Pibuvik configurations. P1: odd sizes throughout (no size a multiple of 16; a latent layer
# with a window shorter than a page, a second one that reads the first one's latent through a window
# longer than a page with other head sizes; grouped keys; a recurrence of three blocks and one of a
# single block and a single tap; layers without a feed-forward). P2: head sizes 64 so that bfloat16
# runs the tensor-core products and the tiled attention kernels with sinks and the temperature; a
# window of exactly one page. P3: nothing optional (no feed-forward, no temperature, no mask, no
# scales), as many key heads as query heads.
def _dense(ff, limit):
    return dict(kind="dense", ff=ff, limit=limit)


def _latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, window=None, kv_from=None):
    out = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale,
               rot=dict(dims=rot_dim, base=base))
    if window is not None:
        out["mask"] = dict(size=window)
    if kv_from is not None:
        out["kv_from"] = kv_from
    return out


PIBUVIK = {
    "P1": dict(
        config=dict(architecture="Pibuvik", vocab=211, width=72, norm=dict(eps=1e-6), residual_mult=0.7,
                    embedding=dict(scale=1.5), logit_scale=0.3, layers=[
            dict(type="latent_attention", mixer=_latent(3, 12, 6, 10, 20, 28, 0.3, 100.0, window=7), mlp=_dense(40, 0.8)),
            dict(type="attention", mixer=dict(heads=4, kv_heads=2, dim=12, vdim=12, scale=0.4,
                                              q_temp=dict(coef=0.3, every=5)), mlp=None),
            dict(type="rglru", mixer=dict(width=48, blocks=3, conv=3), mlp=_dense(56, 1.5)),
            dict(type="latent_attention", mixer=_latent(2, 8, 6, 16, 20, 12, 0.5, 100.0, window=70, kv_from=0), mlp=None),
            dict(type="rglru", mixer=dict(width=40, blocks=1, conv=1), mlp=None),
        ]), seed=31, std=0.12),
    "P2": dict(
        config=dict(architecture="Pibuvik", vocab=512, width=320, norm=dict(eps=2e-5), residual_mult=0.4,
                    embedding=dict(scale=2.0), logit_scale=0.5, layers=[
            dict(type="attention", mixer=dict(heads=8, kv_heads=2, dim=64, vdim=64, scale=0.125,
                                              q_temp=dict(coef=0.25, every=48)), mlp=_dense(384, 2.0)),
            dict(type="rglru", mixer=dict(width=256, blocks=4, conv=4), mlp=_dense(384, 2.0)),
            dict(type="latent_attention", mixer=_latent(4, 64, 32, 64, 96, 128, 0.1, 10000.0, window=100), mlp=_dense(384, 2.0)),
            dict(type="latent_attention", mixer=_latent(4, 32, 32, 32, 96, 64, 0.15, 10000.0, window=64, kv_from=2), mlp=None),
        ]), seed=32, std=0.06),
    "P3": dict(
        config=dict(architecture="Pibuvik", vocab=300, width=64, norm=dict(eps=1e-5), layers=[
            dict(type="rglru", mixer=dict(width=64, blocks=2, conv=2), mlp=None),
            dict(type="attention", mixer=dict(heads=2, kv_heads=2, dim=24, vdim=24, scale=0.2), mlp=None),
            dict(type="latent_attention", mixer=_latent(1, 16, 8, 24, 12, 16, 0.25, 50.0), mlp=None),
        ]), seed=33, std=0.15),
}


def make_pibuvik_dir(path, name, dtype=torch.bfloat16):
    """A model folder of a tiny Pibuvik configuration (a name of PIBUVIK, or a spec of the caller's
    own) with seeded random weights. Norm weights are N(1, 0.2); biases, sinks and the other
    vectors N(0, 0.5); the recurrence's rates N(-3, 1), so that some channels forget at once and
    others carry their state over hundreds of tokens."""
    from llama_rs_metal_b200.engine.model import DecoderModel
    from llama_rs_metal_b200.registry import find_architecture
    from llama_rs_metal_b200.runtime import Runtime
    from llama_rs_metal_b200.weights.random_init import random_tensors, write_model_folder
    spec = PIBUVIK[name] if isinstance(name, str) else name
    arch = find_architecture(spec["config"])
    config = arch.config_class.from_dict(spec["config"])
    model = DecoderModel(arch.plan(config), Runtime(torch.device("cpu"), torch.float32))
    tensors = random_tensors(model.tensor_specs(), spec["seed"], std=spec["std"], vector_mean=0.0, vector_std=0.5,
                             dtype=dtype)
    for name_, t in tensors.items():
        if "norm" in name_.rsplit(".", 1)[-1]:
            t.mul_(0.4).add_(1.0)
        if name_.endswith(".lam"):   # decays from about 0.3 to 0.97 per token: some channels remember far back
            t.mul_(2.0).sub_(3.0)
    return write_model_folder(path, config.to_dict(), tensors, spec["seed"])


def _ssm(heads, vdim, state, groups, conv, norm_groups):
    return dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups)


def _sink_latent(heads, dim, rot_dim, vdim, kv_rank, scale, base):
    return dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale,
                rot=dict(dims=rot_dim, base=base))


def _memory(heads, dim, vdim, cap):
    return dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap)


def _experts(ff, experts, top, identity=0, groups=None, shared=None):
    router = dict(experts=experts, top=top, identity=identity)
    if groups is not None:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    out = dict(kind="moe", expert=dict(ff=ff), router=router)
    if shared is not None:
        out["shared"] = dict(ff=shared)
    return out


def _plain_ff(ff):
    return dict(kind="dense", ff=ff)


# Three tiny Norevik configurations. Between them: state sizes other than the value size, head
# sizes other than the value size, norm parts other than the key groups, one group and several,
# one, two and three kept groups, no identity expert, one, and three, a router without groups and
# without a shared expert, a single chosen expert, layers without a feed-forward, one tap.
NOREVIK = {
    "N1": dict(
        config=dict(architecture="Norevik", vocab=211, width=72, norm=dict(eps=1e-6), embedding=dict(scale=3.0), layers=[
            dict(type="mamba2", mixer=_ssm(4, 12, 20, 2, 3, 4), mlp=_plain_ff(56)),
            dict(type="latent_attention", mixer=_sink_latent(3, 12, 6, 10, 20, 0.3, 100.0),
                 mlp=_experts(24, 5, 2, identity=1, groups=(3, 2), shared=40)),
            dict(type="mlstm", mixer=_memory(3, 8, 20, 6.0), mlp=_experts(16, 4, 3)),
            dict(type="mamba2", mixer=_ssm(2, 24, 8, 1, 1, 1), mlp=None),
            dict(type="latent_attention", mixer=_sink_latent(1, 16, 8, 24, 12, 0.25, 50.0), mlp=None),
        ]), seed=41, std=0.12),
    "N2": dict(
        config=dict(architecture="Norevik", vocab=512, width=256, norm=dict(eps=2e-5), embedding=dict(scale=8.0), layers=[
            dict(type="mlstm", mixer=_memory(4, 64, 32, 15.0), mlp=_experts(64, 13, 4, identity=3, groups=(4, 3), shared=96)),
            dict(type="latent_attention", mixer=_sink_latent(4, 64, 32, 64, 96, 0.1, 10000.0), mlp=_plain_ff(384)),
            dict(type="mamba2", mixer=_ssm(8, 32, 64, 4, 4, 2), mlp=_experts(128, 6, 1, identity=2, groups=(2, 1))),
            dict(type="mlstm", mixer=_memory(2, 32, 96, 8.0), mlp=None),
        ]), seed=42, std=0.06),
    "N3": dict(
        config=dict(architecture="Norevik", vocab=300, width=64, norm=dict(eps=1e-5), layers=[
            dict(type="latent_attention", mixer=_sink_latent(2, 8, 4, 12, 16, 0.35, 30.0), mlp=None),
            dict(type="mlstm", mixer=_memory(1, 16, 16, 10.0), mlp=None),
            dict(type="mamba2", mixer=_ssm(3, 16, 12, 3, 2, 3), mlp=_experts(32, 3, 2, shared=24)),
        ]), seed=43, std=0.15),
}


def make_norevik_dir(path, name, dtype=torch.bfloat16, edit=None, steady_routing=False):
    """A model folder of a tiny Norevik configuration (a name of NOREVIK, or a spec of the caller's
    own) with seeded random weights; `edit` (a function of the name -> tensor dict) may change them
    before they are written. The choice of experts is a step function of the router's input: with
    random weights a runner-up now and then comes within a rounding of bfloat16 activations of the
    last chosen expert, and the engine and the float64 implementation then choose differently.
    `steady_routing` is for comparisons in bfloat16: the corrections are 0, 2, 4, ..., so the same
    experts win for every token (their weights, the scores, still depend on the token) and no
    comparison rests on a close call. Norm weights are N(1, 0.2); biases, sinks, corrections and the
    other vectors N(0, 0.5). The state-space mixer's A_log is N(-2, 1) and the matrix memory's
    forget bias N(2, 1): some heads forget within a few tokens, others carry their state over
    hundreds."""
    from llama_rs_metal_b200.engine.model import DecoderModel
    from llama_rs_metal_b200.registry import find_architecture
    from llama_rs_metal_b200.runtime import Runtime
    from llama_rs_metal_b200.weights.random_init import random_tensors, write_model_folder
    spec = NOREVIK[name] if isinstance(name, str) else name
    arch = find_architecture(spec["config"])
    config = arch.config_class.from_dict(spec["config"])
    model = DecoderModel(arch.plan(config), Runtime(torch.device("cpu"), torch.float32))
    tensors = random_tensors(model.tensor_specs(), spec["seed"], std=spec["std"], vector_mean=0.0, vector_std=0.5,
                             dtype=dtype)
    for name_, t in tensors.items():
        last = name_.rsplit(".", 1)[-1]
        if last in ("norm", "norm1", "norm2"):
            t.mul_(0.4).add_(1.0)
        elif last == "A_log":
            t.mul_(2.0).sub_(2.0)
        elif name_.endswith(".f.b"):
            t.mul_(2.0).add_(2.0)
        elif last == "correction" and steady_routing:
            t.copy_(2.0 * torch.arange(t.numel()))
    if edit is not None:
        edit(tensors)
    return write_model_folder(path, config.to_dict(), tensors, spec["seed"])


def _delta(heads, dim, rank):
    return dict(heads=heads, dim=dim, decay_rank=rank)


def _masked(heads, kv_heads, dim, vdim, scale, rot_dims, base, size, conv=None):
    out = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, rot=dict(dims=rot_dims, base=base),
               mask=dict(size=size))
    if conv is not None:
        out["conv"] = conv
    return out


def _scored_experts(ff, experts, top, scale=None, groups=None, shared=None):
    router = dict(experts=experts, top=top)
    if scale is not None:
        router["scale"] = scale
    if groups is not None:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    out = dict(kind="moe", expert=dict(ff=ff), router=router)
    if shared is not None:
        out["shared"] = dict(ff=shared)
    return out


# Three tiny Tarupel configurations. Between them: odd sizes everywhere (T1), a loop in the middle
# three times, at the start, and none; head sizes 64 and 128 so that bfloat16 takes the tensor-core
# attention kernels (T2) and others that take the row-wise one; values wider and narrower than keys;
# one key head, as many as query heads, and groups; chunks and windows shorter than a page, of one
# page, and longer; a window and a chunk of one position; one tap and five; rotation of the whole
# head and of a part; routers with and without groups, with every expert chosen, without a shared
# expert, without a scale; layers without a feed-forward; residual factors 1 and others.
TARUPEL = {
    "T1": dict(
        config=dict(architecture="Tarupel", vocab=211, width=72, norm=dict(eps=1e-6), embedding=dict(scale=3.0),
                    residual_mult=0.7, loop=dict(start=1, stop=3, times=3), layers=[
            dict(type="attention_2", mixer=_masked(3, 1, 12, 20, 0.3, 6, 100.0, 7), mlp=dict(kind="dense", ff=56)),
            dict(type="general_delta", mixer=_delta(3, 20, 5), mlp=_scored_experts(24, 6, 2, 2.5, (3, 2), 40)),
            dict(type="attention", mixer=_masked(4, 2, 24, 10, 0.25, 24, 50.0, 70, conv=3), mlp=None),
            dict(type="attention", mixer=_masked(2, 2, 10, 10, 0.4, 4, 1000.0, 1, conv=1), mlp=_scored_experts(16, 4, 4)),
            dict(type="general_delta", mixer=_delta(1, 36, 3), mlp=None),
        ]), seed=51, std=0.12),
    "T2": dict(
        config=dict(architecture="Tarupel", vocab=512, width=192, norm=dict(eps=2e-5), embedding=dict(scale=8.0),
                    residual_mult=0.8, loop=dict(start=0, stop=2, times=2), layers=[
            dict(type="attention", mixer=_masked(4, 2, 64, 64, 0.11, 32, 10000.0, 64, conv=2),
                 mlp=_scored_experts(80, 12, 3, 2.0, (4, 2), 112)),
            dict(type="general_delta", mixer=_delta(3, 64, 8), mlp=dict(kind="dense", ff=448)),
            dict(type="attention_2", mixer=_masked(2, 1, 128, 128, 0.09, 64, 500000.0, 100), mlp=_scored_experts(128, 6, 1, 0.5, (2, 1))),
            dict(type="attention_2", mixer=_masked(8, 8, 32, 32, 0.2, 32, 10000.0, 64), mlp=None),
        ]), seed=52, std=0.06),
    "T3": dict(
        config=dict(architecture="Tarupel", vocab=300, width=64, norm=dict(eps=1e-5), layers=[
            dict(type="attention", mixer=_masked(2, 1, 16, 24, 0.3, 8, 30.0, 33, conv=5), mlp=None),
            dict(type="attention_2", mixer=_masked(2, 2, 8, 8, 0.35, 2, 30.0, 1), mlp=dict(kind="dense", ff=40)),
            dict(type="general_delta", mixer=_delta(2, 16, 4), mlp=_scored_experts(32, 3, 2, shared=24)),
        ]), seed=53, std=0.15),
}

STEADY_CHANNEL = 0  # the channel a steadily routed Tarupel folder keeps constant


def make_tarupel_dir(path, name, dtype=torch.bfloat16, edit=None, steady_routing=False):
    """A model folder of a tiny Tarupel configuration (a name of TARUPEL, or a spec of the caller's
    own) with seeded random weights; `edit` (a function of the name -> tensor dict) may change them
    before they are written. Norm weights (single numbers) and the read-out norm's are N(1, 0.2),
    layer scales N(1, 0.3), the shift's mix uniform in [0, 1], biases and the other vectors N(0, 0.5),
    the decay's bias N(0, 2): some channels forget within a few tokens, others carry far.
    The choice of experts is a step function of the router's input: with random weights a
    runner-up now and then comes within a rounding of bfloat16 activations of the last chosen
    expert, and the engine and the float64 implementation then choose differently.
    `steady_routing` is for comparisons in bfloat16: one channel of the stream is the same large
    number for every token (the embedding puts it there, no sublayer adds to it) and the routers
    weigh it by 0, 0.5, 1, ... per expert and everything else a fifth as much, so the same experts win for every token (their weights, the
    scores, still depend on the token) and no comparison rests on a close call."""
    from llama_rs_metal_b200.engine.model import DecoderModel
    from llama_rs_metal_b200.registry import find_architecture
    from llama_rs_metal_b200.runtime import Runtime
    from llama_rs_metal_b200.weights.random_init import _generator, random_tensors, write_model_folder
    spec = TARUPEL[name] if isinstance(name, str) else name
    arch = find_architecture(spec["config"])
    config = arch.config_class.from_dict(spec["config"])
    model = DecoderModel(arch.plan(config), Runtime(torch.device("cpu"), torch.float32))
    tensors = random_tensors(model.tensor_specs(), spec["seed"], std=spec["std"], vector_mean=0.0, vector_std=0.5,
                             dtype=dtype)
    scale = config.embedding_scale
    for name_, t in tensors.items():
        last = name_.rsplit(".", 1)[-1]
        if last in ("norm", "norm1", "norm2"):
            t.mul_(0.4).add_(1.0)
        elif last in ("ls1", "ls2"):
            t.mul_(0.6).add_(1.0)
            if steady_routing:
                t[STEADY_CHANNEL] = 0.0
        elif last == "shift":
            t.copy_(torch.rand(t.shape, generator=_generator(spec["seed"], name_), dtype=torch.float32))
        elif last == "w0":
            t.mul_(4.0)
        elif steady_routing and name_ == "embed":
            t[:, STEADY_CHANNEL] = 4.0 * spec["std"] * 4.0   # several times a typical entry, before the scale
        elif steady_routing and name_ == "loop.step":
            t[:, STEADY_CHANNEL] = 0.0
        elif steady_routing and last == "router":
            t.mul_(0.2)
            t[:, STEADY_CHANNEL] = 0.5 * torch.arange(t.shape[0])
    if edit is not None:
        edit(tensors)
    return write_model_folder(path, config.to_dict(), tensors, spec["seed"])


def random_tokens(seed, length, vocab):
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, vocab, size=length)]


# --------------------------------------------------------------------------- tolerances
# Error is measured against the largest |logit| of the reference rows compared.
#  float32: the engine's sums are float32 in another order than the oracle's float64;
#           a few 1e-6 relative per layer.
#  bfloat16: activations and cache are rounded to 8 bits of mantissa (2^-9 relative)
#           between kernels; a few rounding steps per layer add up to about a percent.
TOLERANCE = {"float32": 2e-5, "bfloat16": 3e-2}


def assert_logits_close(got, ref, dtype, what=""):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.all(np.isfinite(got)), f"{what}: non-finite logits"
    scale = max(float(np.abs(ref).max()), 1e-30)
    err = np.abs(got - ref).max(axis=-1) / scale
    worst = int(err.argmax())
    assert err[worst] <= TOLERANCE[dtype], (
        f"{what}: row {worst} is off by {err[worst]:.3e} of the largest logit "
        f"(allowed {TOLERANCE[dtype]:.1e}); first wrong row "
        f"{int(np.argmax(err > TOLERANCE[dtype]))}")


# --------------------------------------------------------------------------- sampling twin
def gumbel_twin(logits, temperature, seed, key):
    """The device sampler's perturbed scores, restated on the CPU with the same integer hash
    (csrc/sampling.cu): the chosen id is the argmax of what this returns."""
    import math
    mask = (1 << 64) - 1

    def mix(z):
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        return z ^ (z >> 31)
    scores = []
    for i, v in enumerate(logits):
        z = mix((mix((seed + 0x9E3779B97F4A7C15 * (key + 1)) & mask) + i) & mask)
        u = (float(z >> 40) + 0.5) / 16777216.0
        scores.append(float(v) / temperature - math.log(-math.log(u)))
    return scores


# --------------------------------------------------------------------------- traces
class Trace:
    """Steps for bin/trace_run plus, for each step, which (request, position) each row is."""

    def __init__(self):
        self.steps = []
        self.rows = {}

    def add(self, entries, end=()):
        """entries: list of (request id, tokens, first position, want places)."""
        step = len(self.steps)
        self.steps.append({"step": step, "end": list(end), "entries": [
            {"id": rid, "tokens": list(tokens), "want": list(want)} for rid, tokens, _, want in entries]})
        rows = [(rid, first + p) for rid, _, first, want in entries for p in want]
        if rows:
            self.rows[step] = rows
        return step

    def whole(self, name, tokens):
        self.add([(name, tokens, 0, range(len(tokens)))], end=[name])

    def tail_one_by_one(self, name, tokens, tail=32):
        head = max(1, len(tokens) - tail)
        self.add([(name, tokens[:head], 0, range(head))], end=[name] if head == len(tokens) else [])
        for p in range(head, len(tokens)):
            self.add([(name, [tokens[p]], p, [0])], end=[name] if p == len(tokens) - 1 else [])

    def chunks(self, name, tokens, sizes):
        """The sequence in portions: `sizes` is a list of portion lengths (the last one repeats
        until the tokens run out), each portion a step of its own onto the started sequence."""
        at, i = 0, 0
        while at < len(tokens):
            n = min(sizes[min(i, len(sizes) - 1)], len(tokens) - at)
            self.add([(name, tokens[at:at + n], at, range(n))], end=[name] if at + n == len(tokens) else [])
            at, i = at + n, i + 1

    def batch(self, requests, prompt_lengths):
        """requests: {name: tokens}. Prompts (the first prompt_lengths[name] tokens) in one
        step, then one token each per step; a request ends after its last token."""
        names = list(requests)
        done_at = {n: len(requests[n]) for n in names}
        at = {n: prompt_lengths[n] for n in names}
        entries = [(n, requests[n][:at[n]], 0, range(at[n])) for n in names]
        self.add(entries, end=[n for n in names if at[n] == done_at[n]])
        live = [n for n in names if at[n] < done_at[n]]
        while live:
            entries = [(n, [requests[n][at[n]]], at[n], [0]) for n in live]
            for n in live:
                at[n] += 1
            self.add(entries, end=[n for n in live if at[n] == done_at[n]])
            live = [n for n in live if at[n] < done_at[n]]


def run_trace(model_dir, dtype, trace, max_tokens, out_dir, timeout=900):
    """Drive bin/trace_run step by step (next step only after `done`); {step: float32 [rows, vocab]}."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for step in trace.steps:
            proc.stdin.write(json.dumps(step) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {step['step']}", f"trace_run answered {line!r} to step {step['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=timeout) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    with open(os.path.join(model_dir, "config.json")) as handle:
        config = json.load(handle)
        vocab = config["vocab_size"] if "vocab_size" in config else config["vocab"]
    out = {}
    for step, rows in trace.rows.items():
        data = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4")
        assert data.size == len(rows) * vocab, f"step {step}: {data.size} floats for {len(rows)} rows"
        out[step] = data.reshape(len(rows), vocab)
    return out


def check_trace(trace, outputs, reference_logits, dtype):
    """reference_logits: {request: float64 [T, vocab]} from the plain implementation; a trace
    names a request "<mode>:<request>" so that one request can be replayed in several ways."""
    for step in sorted(trace.rows):
        rows = trace.rows[step]
        ref = np.stack([reference_logits[rid.split(":")[-1]][pos] for rid, pos in rows])
        assert_logits_close(outputs[step], ref, dtype,
                            what=f"step {step} ({rows[0][0]} pos {rows[0][1]} ..)")


# --------------------------------------------------------------------------- parity at large widths
_PLAIN_ROWS = {}


def narrowed_copy(model_dir, out_dir, layers):
    """A model folder with the first `layers` layers of `model_dir`: its config.json with
    num_hidden_layers lowered and a link to the same model.safetensors (the loader skips the
    tensors of the layers the smaller model has no use for)."""
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json")) as handle:
        config = json.load(handle)
    config["num_hidden_layers"] = layers
    with open(os.path.join(out_dir, "config.json"), "w") as handle:
        json.dump(config, handle)
    link = os.path.join(out_dir, "model.safetensors")
    if os.path.lexists(link):
        os.remove(link)
    os.symlink(os.path.abspath(os.path.join(model_dir, "model.safetensors")), link)
    return out_dir


def parity_with_plain(engine, model_dir, dtype, prompt_lengths=(300, 170, 40), decode_steps=8, seed=5,
                      chunk=64, keep=4):
    """Run the engine on a model folder in three ways and compare with the plain implementation:
    every prompt alone and whole; all prompts as one batch of unequal lengths followed by
    `decode_steps` steps of one (given, random) token each; the first prompt in portions of
    `chunk` tokens. Logits are compared at each prompt's first position and last `keep` positions
    and at every decoded position. Returns the largest error as a fraction of the largest
    reference logit (assert_logits_close's measure); raises AssertionError beyond the tolerance.
    Works for models too large for a float64 copy (the plain side reads tensors one at a time)."""
    import plain_llama as P
    from llama_rs_metal_b200.cache import Cache
    from llama_rs_metal_b200.engine.batch import StepEntry
    from llama_rs_metal_b200.engine.session import build_model
    from llama_rs_metal_b200.engine.step import StepRunner
    from llama_rs_metal_b200.runtime import Runtime, parse_dtype

    config, tensors = P.read_model_lazily(model_dir)
    vocab = config["vocab_size"]
    seqs = [random_tokens(seed + i, n + decode_steps, vocab) for i, n in enumerate(prompt_lengths)]

    def places(n):
        return sorted(set([0] + list(range(max(0, n - keep), n))))
    wanted = [places(n) + list(range(n, n + decode_steps)) for n in prompt_lengths]
    key = (os.path.realpath(os.path.join(model_dir, "model.safetensors")), config["num_hidden_layers"],
           tuple(prompt_lengths), decode_steps, seed, keep)
    if key not in _PLAIN_ROWS:  # both dtypes compare with the same rows
        _PLAIN_ROWS[key] = [P.forward(config, tensors, s, rows=w).numpy() for s, w in zip(seqs, wanted)]
    refs = _PLAIN_ROWS[key]

    rt = Runtime(engine.device, parse_dtype(dtype))
    _, _, model, _ = build_model(model_dir, rt)
    budget = sum(-(-(n + decode_steps) // 64) * 64 for n in prompt_lengths)
    cache = Cache(model.cache_requests(), rt.dtype, rt.device, budget, len(seqs), max(len(s) for s in seqs))
    runner = StepRunner(model, cache, rt)
    worst = 0.0

    def compare(got, ref, what):
        nonlocal worst
        assert_logits_close(got, ref, dtype, what)
        scale = max(float(np.abs(ref).max()), 1e-30)
        worst = max(worst, float(np.abs(np.asarray(got, dtype=np.float64) - ref).max()) / scale)

    for b, (s, n) in enumerate(zip(seqs, prompt_lengths)):                 # alone and whole
        slot = cache.open_slot()
        out = runner.step([StepEntry(slot, s[:n], places(n))]).cpu().numpy()
        compare(out, refs[b][:len(places(n))], f"prompt {b} alone")
        cache.close_slot(slot)
    slots = [cache.open_slot() for _ in seqs]                              # unequal batch, then decoding
    out = runner.step([StepEntry(sl, s[:n], places(n)) for sl, s, n in zip(slots, seqs, prompt_lengths)]).cpu().numpy()
    row = 0
    for b, n in enumerate(prompt_lengths):
        compare(out[row:row + len(places(n))], refs[b][:len(places(n))], f"prompt {b} in the batch")
        row += len(places(n))
    for step in range(decode_steps):
        out = runner.step([StepEntry(sl, [s[n + step]], [0]) for sl, s, n in zip(slots, seqs, prompt_lengths)])
        out = out.cpu().numpy()
        for b, n in enumerate(prompt_lengths):
            compare(out[b:b + 1], refs[b][len(places(n)) + step][None], f"sequence {b}, decode step {step}")
    for sl in slots:
        cache.close_slot(sl)
    slot, n = cache.open_slot(), prompt_lengths[0]                          # the first prompt in portions
    rows = {}
    for at in range(0, n, chunk):
        m = min(chunk, n - at)
        want = [p - at for p in places(n) if at <= p < at + m]
        out = runner.step([StepEntry(slot, seqs[0][at:at + m], want)]).cpu().numpy()
        for i, p in enumerate(want):
            rows[p + at] = out[i]
    compare(np.stack([rows[p] for p in places(n)]), refs[0][:len(places(n))], f"prompt 0 in portions of {chunk}")
    cache.close_slot(slot)
    runner.check_device_status()
    return worst
