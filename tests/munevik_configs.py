"""Small Munevik configurations for the tests.  Between them they vary every size and option: layer order, a layer without
a feed-forward, latent caches read by later layers with other windows, windows of 1 and wider than any prompt, groups of
one expert, one group, one chosen expert, no shared expert, a recurrent width other than the model's, one block, one tap."""


def attention_layer(heads, dim, rot_dim, vdim, kv_rank, window, mlp, base=10000.0, kv_from=None, scale=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "mask": {"size": window},
             "rot": {"base": base, "dims": rot_dim}, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def recurrent_layer(width, blocks, conv, mlp):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}, "mlp": mlp}


def dense_mlp(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe_mlp(experts, groups, keep, top, ff, scale, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff},
         "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}, "scale": scale}}
    if shared is not None:
        f["shared"] = {"ff": shared}
    return f


MUN_A = {"architecture": "Munevik", "vocab": 97, "width": 64, "postln_alpha": 2.0, "norm": {"eps": 1e-6}, "layers": [
    attention_layer(4, 16, 8, 24, 40, 24, dense_mlp(96, 1.2)),
    recurrent_layer(64, 4, 4, moe_mlp(8, 4, 3, 2, 32, 2.0, shared=48)),
    attention_layer(4, 16, 8, 24, 40, 24, moe_mlp(8, 4, 3, 2, 32, 2.0, shared=48), kv_from=0),
]}

MUN_B = {"architecture": "Munevik", "vocab": 131, "width": 48, "postln_alpha": 1.0, "norm": {"eps": 1e-5}, "layers": [
    recurrent_layer(72, 3, 2, None),
    attention_layer(3, 12, 4, 8, 20, 5, moe_mlp(6, 6, 2, 1, 24, 0.7), base=300.0),
    attention_layer(2, 10, 4, 14, 20, 19, dense_mlp(40, 0.5), base=300.0, kv_from=1, scale=0.4),
    recurrent_layer(48, 1, 1, dense_mlp(56, 3.0)),
]}

MUN_C = {"architecture": "Munevik", "vocab": 64, "width": 80, "postln_alpha": 0.5, "norm": {"eps": 1e-3}, "layers": [
    attention_layer(1, 32, 16, 32, 48, 300, moe_mlp(4, 1, 1, 3, 16, 1.0, shared=8), base=500000.0),
    attention_layer(5, 8, 2, 16, 14, 1, dense_mlp(64, 1.0)),
    recurrent_layer(80, 2, 5, moe_mlp(9, 3, 2, 4, 20, 3.0)),
]}

# cache rows of 128 values and 8 heads: prompt portions of 32 tokens and more take the tensor-core attention kernels in bfloat16
MUN_D = {"architecture": "Munevik", "vocab": 200, "width": 128, "postln_alpha": 1.5, "norm": {"eps": 1e-6}, "layers": [
    attention_layer(8, 32, 16, 32, 112, 64, moe_mlp(4, 2, 2, 2, 48, 1.0, shared=32)),
    recurrent_layer(128, 2, 3, dense_mlp(160, 2.0)),
    attention_layer(8, 32, 16, 32, 112, 33, None, kv_from=0),
]}

# cache rows of 256 values: every attention step takes the head-size-256 tensor-core kernel in bfloat16
MUN_E = {"architecture": "Munevik", "vocab": 150, "width": 96, "postln_alpha": 2.0, "norm": {"eps": 1e-6}, "layers": [
    attention_layer(4, 24, 24, 16, 232, 40, dense_mlp(64, 1.0)),
    attention_layer(2, 24, 24, 40, 232, 77, None, kv_from=0),
]}

# sizes that are multiples of nothing: odd widths, a cache row of 137 values (padded to 144: the general attention kernel in
# both dtypes), blocks of 10 channels, a vocabulary of 101
MUN_F = {"architecture": "Munevik", "vocab": 101, "width": 50, "postln_alpha": 3.0, "norm": {"eps": 1e-5}, "layers": [
    attention_layer(3, 10, 6, 7, 131, 11, moe_mlp(3, 3, 3, 2, 19, 1.3, shared=9), base=77.0),
    recurrent_layer(50, 5, 3, dense_mlp(33, 0.7)),
]}

# recurrent layers only (no pages at all), and attention layers only (each with a cache of its own)
MUN_G = {"architecture": "Munevik", "vocab": 80, "width": 32, "postln_alpha": 1.0, "norm": {"eps": 1e-6}, "layers": [
    recurrent_layer(32, 2, 3, dense_mlp(48, 2.0)), recurrent_layer(64, 64, 2, None)]}
MUN_H = {"architecture": "Munevik", "vocab": 80, "width": 32, "postln_alpha": 1.0, "norm": {"eps": 1e-6}, "layers": [
    attention_layer(2, 8, 8, 8, 24, 16, None), attention_layer(4, 4, 4, 12, 12, 3, dense_mlp(48, 2.0))]}

# a cache row wider than any tensor-core attention kernel takes (300 + 12 values, padded to 320): the general kernel
MUN_I = {"architecture": "Munevik", "vocab": 90, "width": 64, "postln_alpha": 1.0, "norm": {"eps": 1e-6}, "layers": [
    attention_layer(3, 20, 12, 24, 300, 50, dense_mlp(48, 1.0)),
    attention_layer(2, 16, 12, 16, 300, 9, None, kv_from=0),
]}
