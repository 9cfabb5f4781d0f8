"""Small Pedotar configurations for the tests.  They differ from each other in every size, in the order of the layer
types, in which layers have a feed-forward, and in the repeated span; they use values that are easy to get wrong when
two of them happen to be equal elsewhere: key/value heads fewer than heads (and one), values wider and narrower than
keys, chunks that are no multiple of the page size, one to four convolution taps, more states than a warp has lanes
per channel, a span that starts after the first layer and ends before the last, and a configuration without one."""
import copy


def _scan(inner, state, conv, dt_rank, ff=None):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "conv": conv, "dt_rank": dt_rank},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _latent(heads, dim, rot_dim, vdim, rank, base, scale, ff=None, dims=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
                      "rot": {"base": base, "dims": rot_dim if dims is None else dims}},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _chunked(heads, kv_heads, dim, vdim, size, scale, ff=None):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size}},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


P1 = {"architecture": "Pedotar", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "kv_page_size": 4,
      "layers": [_chunked(6, 2, 16, 24, 5, 0.3), _scan(80, 5, 4, 3, ff=64), _latent(3, 8, 8, 12, 20, 100.0, 0.4)],
      "loop": {"start": 1, "stop": 3, "times": 3}}

P2 = {"architecture": "Pedotar", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}, "kv_page_size": 8,
      "layers": [_latent(4, 16, 4, 16, 24, 10000.0, 0.3, ff=48), _scan(128, 16, 2, 8), _chunked(4, 1, 32, 8, 33, 0.25, ff=40),
                 _scan(64, 40, 1, 1, ff=72)]}

# widths at which the bfloat16 path takes its tensor-core products (multiples of 8 and 16 throughout)
P3 = {"architecture": "Pedotar", "vocab": 512, "width": 128, "norm": {"eps": 1e-6}, "kv_page_size": 16,
      "layers": [_scan(256, 16, 4, 8), _chunked(4, 2, 32, 64, 48, 0.2, ff=192), _latent(4, 32, 16, 48, 64, 50000.0, 0.15, ff=192),
                 _chunked(8, 8, 16, 16, 100, 0.3)],
      "loop": {"start": 0, "stop": 2, "times": 2}}

# nothing a multiple of 4: every product, norm and attention on its general path
P4 = {"architecture": "Pedotar", "vocab": 131, "width": 50, "norm": {"eps": 1e-5}, "kv_page_size": 3,
      "layers": [_scan(30, 3, 2, 2), _latent(2, 6, 2, 5, 7, 1000.0, 0.4, ff=22), _chunked(2, 1, 6, 10, 9, 0.4)],
      "loop": {"start": 0, "stop": 3, "times": 2}}

ALL = {"P1": P1, "P2": P2, "P3": P3, "P4": P4}


def get(name):
    return copy.deepcopy(ALL[name])


def one_layer(layer, width=48, vocab=101, page=4, eps=1e-5):
    """A model of a single layer: one mechanism alone between the embedding and the head."""
    return {"architecture": "Pedotar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "kv_page_size": page,
            "layers": [copy.deepcopy(layer)]}


scan, latent, chunked = _scan, _latent, _chunked
