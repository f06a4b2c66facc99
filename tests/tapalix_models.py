"""Small Tapalix configurations for the tests, and folders of random weights for them.

The configurations differ from one another in every size and option: query, turned and value
widths that differ from each other, ranks below and above the head size, a turned part of which
only some columns turn, rotation with and without stretched frequencies, one head, one expert per
group, a single group, top 1, layers without feed-forward or without a shared expert, a loop over
the first layers, over the last ones, of a single pass and none at all, logits without a cap, an
embedding that is not scaled, widths that are no multiple of eight.
"""

from __future__ import annotations

from pathlib import Path

import torch


def scaling(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def latent(heads, dim, rot_dim, vdim, rank, scale=None, base=10000.0, rot_dims=None, stretch=None):
    return {"type": "latent_attention", "mixer": {
        "heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
        "scale": (dim + rot_dim) ** -0.5 if scale is None else scale,
        "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims, "scaling": stretch}}}


def gated(heads, dim, vdim, rank, scale=None):
    return {"type": "latent_attention_2", "mixer": {
        "heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank,
        "scale": dim ** -0.5 if scale is None else scale}}


def moe(ff, experts, top, groups=None, scale=1.0, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router,
            "shared": None if shared is None else {"ff": shared}}


def with_mlp(layer, mlp):
    layer = dict(layer)
    layer["mlp"] = mlp
    return layer


def model(vocab, width, eps, layers, loop=None, embedding=1.0, logit_scale=1.0, softcap=0.0):
    return {"architecture": "Tapalix", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": embedding}, "logit_scale": logit_scale, "logit_softcap": softcap,
            "loop": None if loop is None else {"start": loop[0], "stop": loop[1], "times": loop[2]},
            "layers": layers}


CONFIGS = {
    # the rotated mixer alone: stretched frequencies whose ramp lies inside the pairs, a turned part
    # of which four of six columns turn, a sharp softmax, no feed-forward, no loop, no cap
    "rotated": model(97, 40, 1e-5, [
        with_mlp(latent(3, 10, 6, 14, 20, scale=1.5, base=50.0, rot_dims=4,
                        stretch=scaling(4.0, 24, 3.0, 1.0)), None)]),
    # the gated mixer alone, with a feed-forward of experts without a shared one and without groups
    "gated": model(83, 48, 1e-6, [
        with_mlp(gated(4, 12, 20, 28, scale=1.2), moe(24, 5, 2, scale=1.5))], softcap=9.0),
    # the experts alone under the simplest mixer: groups of three of which two are kept, top 3,
    # a shared expert, the choice made among negative scores
    "experts": model(71, 32, 1e-6, [
        with_mlp(gated(1, 8, 8, 8), moe(16, 12, 3, groups=(4, 2), scale=2.5, shared=40))],
        embedding=3.0),
    # the loop: two passes over the two middle layers, each pass with its own cache
    "loop": model(131, 64, 1e-6, [
        with_mlp(latent(2, 16, 8, 12, 24, scale=0.5, stretch=scaling(2.0, 64, 8.0, 1.0)), moe(32, 6, 2, groups=(3, 2), shared=24)),
        with_mlp(gated(4, 8, 16, 40, scale=0.7), moe(16, 8, 3, groups=(2, 1), scale=2.0, shared=48)),
        with_mlp(latent(4, 8, 4, 8, 40, scale=0.7, base=100.0), None),
        with_mlp(gated(2, 16, 8, 12), moe(40, 4, 1))],
        loop=(1, 3, 2), embedding=4.0, logit_scale=2.5, softcap=12.0),
    # a loop from the first layer on and of a single pass; a loop up to the last layer
    "loop_first": model(90, 40, 1e-5, [
        with_mlp(gated(2, 8, 8, 16), moe(24, 4, 2, groups=(4, 2))),
        with_mlp(latent(2, 8, 4, 8, 16), None)], loop=(0, 1, 1), logit_scale=0.5),
    "loop_last": model(90, 40, 1e-5, [
        with_mlp(latent(2, 8, 4, 8, 16, stretch=scaling(3.0, 32, 4.0, 2.0)), None),
        with_mlp(gated(2, 8, 8, 16), moe(24, 6, 2, groups=(6, 3), shared=16))], loop=(1, 2, 2),
        softcap=5.0),
    # sizes that are no multiple of eight, single heads, a rank below the head size
    "odd": model(61, 36, 1e-5, [
        with_mlp(latent(1, 6, 2, 10, 5, scale=0.7), moe(10, 3, 1, shared=7)),
        with_mlp(gated(3, 6, 10, 9, scale=0.7), moe(14, 6, 4, groups=(2, 2), scale=0.5))],
        loop=(0, 2, 2), embedding=2.0, softcap=20.0),
    # head sizes of real models in small: eight heads over one latent row, rank 64 and 128, tiles
    # of experts that hold more than one tile's rows
    "wide": model(150, 128, 1e-6, [
        with_mlp(latent(8, 32, 16, 32, 64, stretch=scaling(2.0, 128, 16.0, 1.0)), moe(64, 8, 2, groups=(4, 2), scale=1.5, shared=96)),
        with_mlp(gated(4, 64, 64, 128), moe(32, 16, 4, groups=(4, 3), scale=2.0, shared=64)),
        with_mlp(latent(4, 64, 64, 64, 64, base=5e5), moe(64, 4, 2))],
        loop=(1, 2, 2), embedding=8.0, logit_scale=1.5, softcap=14.0),
}


def write_model(root, name, seed=0, std=0.08, sharpen=True) -> Path:
    """A folder with config.json and random weights for CONFIGS[name].  With `sharpen` the routers'
    corrections are drawn wide (N(0, 1)): choices are then made among negative scores too, and the
    order of the choice differs from the order of the weights; the query and key projections are
    drawn three times as wide, so that scores spread and single keys stand out, and the routers ten
    times as wide, so that every token chooses its own experts.  Without it the routers are drawn
    narrow and the corrections are 4 x 2^k with every k once: the scores lie inside (0, 1), so
    neither two experts' choice values nor two groups' sums of two come closer than 2, the choice
    rests on the corrections alone and no rounding can turn it - which is what a comparison in
    bfloat16 needs; the weights still come from each token's own scores."""
    from from_scratch_inference_engine_b200.config import config_from_dict
    from from_scratch_inference_engine_b200.weights import load_file, save_file, write_random_model

    folder = write_random_model(Path(root) / f"tapalix_{name}", config_from_dict(CONFIGS[name]),
                                seed, std, torch.bfloat16)
    tensors = load_file(folder / "model.safetensors")
    generator = torch.Generator().manual_seed(seed + 1000)
    for key in list(tensors):
        if key.endswith(".correction") and sharpen:
            tensors[key] = torch.randn(tensors[key].shape, generator=generator).to(torch.bfloat16)
        elif key.endswith(".correction"):
            order = torch.randperm(tensors[key].numel(), generator=generator)
            tensors[key] = (4.0 * torch.pow(2.0, order.float())).to(torch.bfloat16)
        elif key.endswith(".router"):
            tensors[key] = (tensors[key].float() * (10.0 if sharpen else 0.3)).to(torch.bfloat16)
        elif sharpen and key.split(".")[-1] in ("q", "dkv", "uk") and ".mix." in key:
            tensors[key] = (tensors[key].float() * 3.0).to(torch.bfloat16)
    save_file(tensors, folder / "model.safetensors")
    return folder
