"""Small Kipedra configurations for the tests.  They differ from each other in every size, in the order of the layer
types, in the kind of feed-forward and in the repeated span, and they use values that are easy to get wrong when two of
them happen to be equal elsewhere: key heads fewer than heads (and one, and as many), values wider and narrower than
keys, windows that are no multiple of the page size (and one position wide), one to five convolution taps, rotations of
none, part and all of a head, one expert per token, a multiplier of one, layers without a feed-forward."""
import copy


def _ff(kind):
    if kind is None:
        return None
    if kind[0] == "dense":
        return {"kind": "dense", "ff": kind[1]}
    _, experts, top, ff, scale = kind
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}


def delta(heads, kv_heads, dim, vdim, conv, ff=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": _ff(ff)}


def attention(heads, kv_heads, dim, vdim, conv, window, dims, base, scale, ff=None):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale, "mask": {"size": window},
                      "rot": {"base": base, "dims": dims}},
            "mlp": _ff(ff)}


def one_layer(layer, width=48, vocab=61, page=4, mult=0.7):
    return {"architecture": "Kipedra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "residual_mult": mult, "kv_page_size": page,
            "layers": [copy.deepcopy(layer)]}


K1 = {"architecture": "Kipedra", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "residual_mult": 0.5, "kv_page_size": 4,
      "layers": [attention(6, 2, 16, 24, 3, 7, 8, 100.0, 0.5, ff=("moe", 5, 2, 40, 2.0)), delta(4, 2, 24, 12, 2, ff=("dense", 64)),
                 delta(3, 3, 8, 40, 4)],
      "loop": {"start": 0, "stop": 2, "times": 3}}

K2 = {"architecture": "Kipedra", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}, "residual_mult": 1.0, "kv_page_size": 8,
      "layers": [delta(2, 1, 32, 16, 1, ff=("moe", 3, 1, 24, 1.0)), attention(4, 4, 16, 16, 1, 33, 16, 10000.0, 0.25, ff=("dense", 48)),
                 attention(4, 1, 32, 8, 5, 9, 0, 10000.0, 0.2), delta(4, 4, 16, 24, 3, ff=("dense", 40))]}

# widths at which the bfloat16 path takes its tensor-core products and attention kernels (multiples of 8 and 16, heads of 64 and 128)
K3 = {"architecture": "Kipedra", "vocab": 384, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.4, "kv_page_size": 16,
      "layers": [delta(4, 2, 64, 48, 4, ff=("dense", 192)), attention(4, 2, 128, 128, 4, 100, 64, 50000.0, 0.09, ff=("moe", 8, 2, 64, 1.5)),
                 attention(8, 2, 64, 64, 2, 48, 64, 1000.0, 0.125, ff=("moe", 16, 4, 32, 2.5)), delta(2, 2, 128, 128, 2)],
      "loop": {"start": 1, "stop": 3, "times": 2}}

# no size a multiple of 4: every product, norm and attention takes its general path
K4 = {"architecture": "Kipedra", "vocab": 33, "width": 50, "norm": {"eps": 1e-5}, "residual_mult": 0.9, "kv_page_size": 3,
      "layers": [attention(3, 1, 10, 6, 2, 5, 6, 300.0, 0.4, ff=("moe", 7, 3, 9, 0.7)), delta(5, 5, 7, 9, 3, ff=("dense", 11)),
                 attention(2, 2, 6, 14, 3, 21, 2, 50.0, 0.3, ff=("dense", 13))],
      "loop": {"start": 1, "stop": 2, "times": 2}}

ALL = {"K1": K1, "K2": K2, "K3": K3, "K4": K4}


def get(name):
    return copy.deepcopy(ALL[name])
