"""Small Pererax configurations for the tests, and the folder writer they share.

A: sizes that share no factor with the kernels' tiles; key and value heads of different sizes on the
left of the pair; a rotation of part of each head; three of five experts plus two identity outputs;
a delta mixer with fewer query/key heads than value heads, three taps and two different inner sizes
of its low-rank pairs; a layer without feed-forward; two layers that run another layer's tensors; a
window that is no multiple of a page.
B: everything a multiple of 8, so that 16-bit runs take the tensor-core products; as many KV heads as
query heads in one attention and one KV head in the other; a window longer than two pages; three of
six experts plus three identity outputs; key size 64 in the recurrences.
C: the smallest of everything: one head, a window of one key, one tap, one expert chosen out of one
plus one identity output, no unit for every token, no soft cap, no rotation on the left of the pair,
a scale of one on the router's weights.
"""
import os

_MLP_A = {"kind": "moe", "expert": {"ff": 20, "limit": 2.5}, "router": {"experts": 5, "identity": 2, "top": 3, "scale": 1.5},
          "shared": {"ff": 28, "limit": 1.5}}
_PAIR_A = {"left": {"heads": 3, "kv_heads": 1, "dim": 10, "vdim": 14, "scale": 0.4, "softcap": 3.0, "rot": {"base": 100.0, "dims": 6}},
           "right": {"heads": 3, "dim": 6, "vdim": 10, "gate_cap": 7.0}}
_DELTA_A = {"heads": 4, "kv_heads": 2, "dim": 10, "vdim": 6, "conv": 3, "decay_rank": 5, "gate_rank": 7}
PERERAX_A = {
    "architecture": "Pererax", "vocab": 197, "width": 52, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "parallel", "mixer": _PAIR_A, "mlp": _MLP_A},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 12, "scale": 0.3, "mask": {"size": 19},
                                        "rot": {"base": 500.0, "dims": 8}}, "mlp": None},
        {"type": "channel_delta", "mixer": _DELTA_A, "mlp": _MLP_A},
        {"type": "parallel", "mixer": _PAIR_A, "mlp": _MLP_A, "weights_of": 0},
        {"type": "channel_delta", "mixer": _DELTA_A, "mlp": _MLP_A, "weights_of": 2},
    ],
}
_MLP_B = {"kind": "moe", "expert": {"ff": 64, "limit": 1.75}, "router": {"experts": 6, "identity": 3, "top": 3, "scale": 1.25},
          "shared": {"ff": 96, "limit": 0.9}}
PERERAX_B = {
    "architecture": "Pererax", "vocab": 256, "width": 128, "norm": {"eps": 3e-6},
    "layers": [
        {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 4, "dim": 64, "vdim": 32, "conv": 4, "decay_rank": 16, "gate_rank": 8},
         "mlp": _MLP_B},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 4, "dim": 32, "vdim": 32, "scale": 0.2, "mask": {"size": 36},
                                        "rot": {"base": 10000.0, "dims": 32}}, "mlp": _MLP_B},
        {"type": "parallel", "mixer": {"left": {"heads": 4, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.18, "softcap": 20.0,
                                                "rot": {"base": 20000.0, "dims": 16}},
                                       "right": {"heads": 2, "dim": 64, "vdim": 40, "gate_cap": 10.0}}, "mlp": _MLP_B},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 4, "dim": 32, "vdim": 32, "scale": 0.2, "mask": {"size": 36},
                                        "rot": {"base": 10000.0, "dims": 32}}, "mlp": _MLP_B, "weights_of": 1},
    ],
}
_MLP_C = {"kind": "moe", "expert": {"ff": 24, "limit": 3.0}, "router": {"experts": 1, "identity": 1, "top": 1}}
PERERAX_C = {
    "architecture": "Pererax", "vocab": 64, "width": 32, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.35, "mask": {"size": 1},
                                        "rot": {"base": 10.0, "dims": 2}}, "mlp": _MLP_C},
        {"type": "channel_delta", "mixer": {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 36, "conv": 1, "decay_rank": 1, "gate_rank": 2},
         "mlp": None},
        {"type": "parallel", "mixer": {"left": {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 6, "scale": 0.5},
                                       "right": {"heads": 1, "dim": 5, "vdim": 33, "gate_cap": 4.0}},
         "mlp": {"kind": "moe", "expert": {"ff": 8, "limit": 1.0}, "router": {"experts": 3, "top": 3, "scale": 0.5}}},
    ],
}
PERERAX = {"A": (PERERAX_A, 3), "B": (PERERAX_B, 4), "C": (PERERAX_C, 5)}


def write_model(cfg, folder, seed, std=0.12):
    """config.json + model.safetensors (bfloat16 matrices, short tensor names) from the engine's
    random-weights mode; the plain implementation reads the folder with its own reader."""
    from ferrum_b200.weights import write_random_model
    write_random_model(cfg, folder, seed, dtype="bfloat16", std=std)
    assert os.path.exists(os.path.join(folder, "model.safetensors"))
    return folder
