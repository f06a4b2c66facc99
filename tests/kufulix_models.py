"""Small Kufulix configurations for the tests, and folders of random weights for them.

The configurations differ from one another in every size and option: key and value widths that
differ, query heads per key/value head from one to three, windows and chunks that are no multiple
of a page, rotation over part of a head, over all of it and none, with and without rescaled
frequencies, state-space mixers with one and two groups, one to four taps, a norm in one and in two
parts, layers without a feed-forward, experts with and without identity experts and groups, top 1,
layers that run another layer's tensors, logits without a cap, widths that are no multiple of eight.
"""

from __future__ import annotations

from pathlib import Path

import torch


def rot(base, dims, scaling=None):
    return {"base": base, "dims": dims,
            "scaling": None if scaling is None else dict(zip(("factor", "low", "high", "original"), scaling))}


def attention(heads, kv_heads, dim, vdim, size, rotation, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size},
            "rot": rotation, "scale": dim ** -0.5 if scale is None else scale}


def state_space(heads, vdim, state, groups=1, conv=4, norm_groups=1):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
            "norm_groups": norm_groups}


def parallel(left, right, left_scale=1.0, right_scale=1.0, mlp=None, **more):
    return dict({"type": "parallel", "mlp": mlp,
                 "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}},
                **more)


def chunked(mixer, mlp=None, **more):
    return dict({"type": "attention", "mixer": mixer, "mlp": mlp}, **more)


def moe(ff, experts, top, identity=0, groups=None):
    router = {"experts": experts, "top": top, "identity": identity}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def again(layer, source):
    """`layer` once more, running the tensors of layer `source`."""
    return dict(layer, weights_of=source)


def model(vocab, width, eps, layers, softcap=0.0):
    return {"architecture": "Kufulix", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "logit_softcap": softcap, "layers": layers}


_WINDOW = parallel(attention(4, 2, 12, 10, 9, rot(50.0, 8, (4.0, 1.0, 4.0, 32))),
                   state_space(3, 8, 6, conv=3), 0.5, 1.5)
_SHARED_A = parallel(attention(3, 3, 16, 8, 21, rot(100.0, 16, (2.0, 1.0, 2.0, 16))),
                     state_space(4, 8, 8, groups=2, conv=4, norm_groups=2), 0.75, 1.25,
                     mlp=moe(24, 6, 2, identity=2, groups=(4, 3)))
_SHARED_B = chunked(attention(4, 2, 8, 16, 13, rot(1000.0, 4), scale=0.5), mlp=moe(16, 5, 3, identity=1))

CONFIGS = {
    # the parallel mixer alone: a window of 9 over pages of 16, two query heads per key/value head,
    # rotation over 8 of 12 columns with rescaled frequencies whose ramp lies inside the pairs,
    # three taps, no feed-forward, no cap
    "window": model(97, 40, 1e-5, [_WINDOW]),
    # the chunked, gated attention alone: chunks of 11, three query heads per key/value head,
    # the whole head rotated, plain frequencies
    "chunk": model(83, 48, 1e-6, [chunked(attention(6, 2, 16, 12, 11, rot(10000.0, 16), scale=0.6))],
                   softcap=9.0),
    # the experts alone under the simplest mixer: six experts and two identity experts in four
    # groups of two of which two are kept, top 3
    "experts": model(71, 32, 1e-6, [chunked(attention(1, 1, 8, 8, 64, None),
                                            mlp=moe(20, 6, 3, identity=2, groups=(4, 2)))], softcap=30.0),
    # layers that run other layers' tensors, each with its own cache and state; a state-space
    # mixer with two groups and a norm in two parts
    "shared": model(131, 64, 1e-6, [_SHARED_A, _SHARED_B, again(_SHARED_A, 0), again(_SHARED_B, 1),
                                    again(_SHARED_A, 0)], softcap=12.0),
    # two taps and one tap (no inputs kept), a single head, top 1 without groups or identity
    # experts, a window of one (a token sees itself only), no rotation
    "plain": model(90, 40, 1e-5, [
        parallel(attention(1, 1, 8, 8, 1, None), state_space(1, 16, 4, conv=1), 2.0, 0.5, mlp=moe(24, 4, 1)),
        parallel(attention(2, 1, 8, 8, 5, rot(20.0, 2)), state_space(2, 4, 12, conv=2), 1.0, 1.0)]),
    # sizes that are no multiple of eight or four
    "odd": model(61, 36, 1e-5, [
        parallel(attention(3, 1, 6, 10, 7, rot(30.0, 6, (8.0, 1.0, 4.0, 8))),
                 state_space(3, 5, 7, groups=3, conv=4, norm_groups=3), 0.6, 1.1, mlp=moe(10, 3, 2, identity=3, groups=(3, 2))),
        chunked(attention(3, 3, 10, 6, 5, rot(500.0, 4)), mlp=moe(14, 7, 4, identity=1, groups=(2, 1)))],
        softcap=20.0),
    # head sizes of real models in small: the tensor-core attention takes the windowed and the
    # chunked layers, long portions take the experts' grouped product
    "wide": model(150, 128, 1e-6, [
        parallel(attention(4, 2, 64, 64, 40, rot(10000.0, 32, (8.0, 1.0, 4.0, 64))),
                 state_space(4, 32, 32, groups=2, conv=4), 0.7, 1.2, mlp=moe(64, 8, 2, identity=4, groups=(3, 2))),
        chunked(attention(4, 1, 64, 64, 48, rot(500000.0, 64, (4.0, 1.0, 4.0, 128))), mlp=moe(32, 4, 2)),
        again(parallel(attention(4, 2, 64, 64, 40, rot(10000.0, 32, (8.0, 1.0, 4.0, 64))),
                       state_space(4, 32, 32, groups=2, conv=4), 0.7, 1.2,
                       mlp=moe(64, 8, 2, identity=4, groups=(3, 2))), 0)],
        softcap=14.0),
}


def write_model(root, name, seed=0, std=0.08, sharpen=True) -> Path:
    """A folder with config.json and random weights for CONFIGS[name].  The state-space mixers'
    decays are spread from slow to fast over the heads (A_log from -4 to 0.5) and their step sizes
    drawn wide, so that some heads remember hundreds of tokens and others a few.  With `sharpen` the
    routers' corrections are spread wide and shuffled (choices are made among negative values too, and
    the order of the choice differs from the order of the weights), the routers four times as wide (every
    token chooses its own experts), and the query and key projections - where they are normed, the
    norms' gains - three times as wide, so that scores spread and single keys stand out.  Without
    it the routers are drawn narrow and the corrections are 4 x 2^k with every k once: no rounding
    can turn a choice, which is what a comparison in bfloat16 needs; the weights still come from
    each token's own scores."""
    from from_scratch_inference_engine_b200.config import config_from_dict
    from from_scratch_inference_engine_b200.weights import load_file, save_file, write_random_model

    folder = write_random_model(Path(root) / f"kufulix_{name}", config_from_dict(CONFIGS[name]),
                                seed, std, torch.bfloat16)
    tensors = load_file(folder / "model.safetensors")
    generator = torch.Generator().manual_seed(seed + 1000)
    for key in list(tensors):
        last = key.split(".")[-1]
        if last == "correction" and sharpen:
            # spread evenly and shuffled: no two experts share a value after rounding to bfloat16 (a
            # shared value would leave the choice between them to score differences below 32-bit rounding)
            count = tensors[key].numel()
            spread = torch.linspace(-0.4, 0.4, count) if count > 1 else torch.zeros(1)
            tensors[key] = spread[torch.randperm(count, generator=generator)].to(torch.bfloat16)
        elif last == "correction":
            order = torch.randperm(tensors[key].numel(), generator=generator)
            tensors[key] = (4.0 * torch.pow(2.0, order.float())).to(torch.bfloat16)
        elif last == "router":
            tensors[key] = (tensors[key].float() * (4.0 if sharpen else 0.3)).to(torch.bfloat16)
        elif last == "A_log":
            tensors[key] = torch.linspace(-4.0, 0.5, tensors[key].numel()).to(torch.bfloat16)
        elif last == "dt_bias":
            tensors[key] = (torch.rand(tensors[key].shape, generator=generator) * 3.0 - 2.0).to(torch.bfloat16)
        elif sharpen and ".mix." in key and (key.endswith(".q.norm") or key.endswith(".k.norm")):
            tensors[key] = (tensors[key].float() * 3.0).to(torch.bfloat16)
        elif sharpen and ".mix." in key and ".left." not in key and last in ("q", "k"):
            tensors[key] = (tensors[key].float() * 3.0).to(torch.bfloat16)
    save_file(tensors, folder / "model.safetensors")
    return folder


def random_config(seed: int) -> dict:
    """A configuration drawn at random: two to five layers of either type, some of them running an
    earlier layer's tensors, every size, mask, rotation, scale and router drawn anew."""
    import random
    rng = random.Random(seed)

    def draw_attention():
        kv_heads = rng.choice([1, 2, 3])
        heads = kv_heads * rng.choice([1, 2, 4])
        dim = rng.choice([6, 8, 16, 24, 32, 64])
        vdim = rng.choice([4, 8, 10, 16, 32, 64])
        dims = rng.choice([0, 2, dim // 2 // 2 * 2, dim // 2 * 2])
        rotation = None
        if dims:
            scaling = rng.choice([None, (rng.choice([2.0, 4.0, 8.0]), 1.0, rng.choice([2.0, 4.0]), rng.choice([8, 16, 64]))])
            rotation = rot(rng.choice([20.0, 1000.0, 500000.0]), dims, scaling)
        return attention(heads, kv_heads, dim, vdim, rng.choice([1, 3, 7, 16, 21, 40, 64, 100]), rotation,
                         scale=rng.choice([None, 0.3, 1.0]))

    def draw_state_space():
        groups = rng.choice([1, 2])
        heads = groups * rng.choice([1, 2, 3])
        vdim = rng.choice([4, 5, 8, 16, 32])
        parts = rng.choice([p for p in (1, 2, 3, 4) if (heads * vdim) % p == 0])
        return state_space(heads, vdim, rng.choice([3, 4, 8, 16, 33]), groups, rng.choice([1, 2, 3, 4]), parts)

    def draw_mlp():
        if rng.random() < 0.2:
            return None
        experts, identity = rng.choice([1, 3, 4, 6, 8]), rng.choice([0, 0, 1, 2, 4])
        routed = experts + identity
        groups = None
        counts = [c for c in (2, 3, 4) if routed % c == 0]
        if counts and rng.random() < 0.6:
            count = rng.choice(counts)
            groups = (count, rng.randint(1, count))
        room = routed if groups is None else groups[1] * (routed // groups[0])
        return moe(rng.choice([8, 12, 16, 40]), experts, rng.randint(1, min(room, 4)), identity, groups)

    layers = []
    for index in range(rng.randint(2, 5)):
        if layers and rng.random() < 0.3:
            source = rng.choice([i for i, layer in enumerate(layers) if "weights_of" not in layer])
            layers.append(again(layers[source], source))
        elif rng.random() < 0.6:
            layers.append(parallel(draw_attention(), draw_state_space(), rng.choice([0.5, 1.0, 1.3]),
                                   rng.choice([0.7, 1.0, 1.5]), mlp=draw_mlp()))
        else:
            layers.append(chunked(draw_attention(), mlp=draw_mlp()))
    return model(rng.choice([50, 97, 128]), rng.choice([24, 36, 64, 128]), rng.choice([1e-5, 1e-6]), layers,
                 softcap=rng.choice([0.0, 8.0, 30.0]))


def write_random(root, seed: int, sharpen=True) -> Path:
    """A folder for `random_config(seed)`, which is entered into CONFIGS as "random<seed>"."""
    CONFIGS[f"random{seed}"] = random_config(seed)
    return write_model(root, f"random{seed}", seed=seed, sharpen=sharpen)
