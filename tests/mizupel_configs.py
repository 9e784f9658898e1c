"""Small Mizupel configurations for the tests: other sizes, orders, windows and constants than any model folder that is served."""


def attn(heads, kv_heads, dim, vdim, scale, conv=None, window=None, rot=None, softcap=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv is not None:
        m["conv"] = conv
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = rot
    if softcap is not None:
        m["softcap"] = softcap
    return m


def layer(kind, mixer, ff=None, weights_of=None):
    L = {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}
    if weights_of is not None:
        L["weights_of"] = weights_of
    return L


SCALED = {"base": 100.0, "dims": 8, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}   # all three frequency bands occur

# every mixer, grouped kv heads, a value size above the key size, a layer that runs another's tensors
_A0 = layer("attention", attn(4, 2, 16, 24, 0.3, conv=3, window=11, rot=SCALED, softcap=20.0), ff=96)
_A2 = layer("wkv", {"heads": 2, "dim": 32, "decay_rank": 8}, ff=80)
MIZ_A = {"architecture": "Mizupel", "vocab": 131, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 10.0, "layers": [
    _A0, layer("mlstm", {"heads": 2, "dim": 16, "vdim": 24, "gate_cap": 8.0}), _A2, dict(_A0, weights_of=0), dict(_A2, weights_of=2)]}

# sizes that are multiples of nothing; full attention without convolution state (one tap), cap or window; every value rotated;
# a key size above the value size; heads x dim other than the width; a key size that fills its last slice of the state partly
MIZ_B = {"architecture": "Mizupel", "vocab": 97, "width": 50, "norm": {"eps": 3e-4}, "logit_softcap": None, "layers": [
    layer("wkv", {"heads": 3, "dim": 12, "decay_rank": 5}),
    layer("attention", attn(3, 3, 10, 6, 0.4, conv=1, rot={"base": 30.0, "dims": 10}), ff=70),
    layer("mlstm", {"heads": 1, "dim": 40, "vdim": 20, "gate_cap": 2.0}, ff=33),
    layer("attention", attn(2, 1, 12, 12, 0.25, window=200, softcap=3.0))]}              # no convolution, no rotation at all

# one kv head under six heads, equal key and value size (no padding), a window of one key, five taps, two rotated values
MIZ_C = {"architecture": "Mizupel", "vocab": 64, "width": 48, "norm": {"eps": 1e-6}, "logit_softcap": 4.0, "layers": [
    layer("attention", attn(6, 1, 32, 32, 0.2, conv=5, window=1, rot={"base": 10.0, "dims": 2}), ff=64),
    layer("attention", attn(6, 1, 32, 32, 0.2, conv=2, window=17, rot={"base": 5000.0, "dims": 32}, softcap=50.0))]}

# recurrent layers only, each kind run twice over the same tensors
_D0 = layer("wkv", {"heads": 1, "dim": 48, "decay_rank": 3}, ff=40)
_D1 = layer("mlstm", {"heads": 3, "dim": 8, "vdim": 36, "gate_cap": 15.0})
MIZ_D = {"architecture": "Mizupel", "vocab": 80, "width": 40, "norm": {"eps": 1e-5}, "logit_softcap": 30.0, "layers": [
    _D0, _D1, dict(_D0, weights_of=0), dict(_D1, weights_of=1)]}

# head sizes the tensor-core attention kernels take (64 and 128 values), with a soft cap and a window
MIZ_E = {"architecture": "Mizupel", "vocab": 120, "width": 128, "norm": {"eps": 1e-5}, "logit_softcap": 12.0, "layers": [
    layer("attention", attn(8, 2, 64, 64, 0.125, conv=4, window=70, rot={"base": 1000.0, "dims": 16}, softcap=8.0), ff=128),
    layer("attention", attn(4, 1, 128, 96, 0.09, conv=2, window=300, rot=dict(SCALED, dims=64), softcap=15.0)),
    layer("wkv", {"heads": 2, "dim": 64, "decay_rank": 16})]}

ALL = {"A": MIZ_A, "B": MIZ_B, "C": MIZ_C, "D": MIZ_D, "E": MIZ_E}
