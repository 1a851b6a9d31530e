"""Small Zavesun configurations for the tests, and the folder writer they share.

A: sizes that share no factor with the kernels' tiles; three streams; key and value heads of
different sizes; the first value-mixing layer is not the first layer; a layer without feed-forward;
two experts per token out of five; a rotation of part of the head at divided frequencies and one
without a scaling block; windows and chunks that are no multiples of a page.
B: everything a multiple of 8, so that 16-bit runs take the tensor-core products; two streams; no
soft cap; one KV head under four query heads and as many KV heads as query heads; four experts per
token out of sixteen and one out of four; a window and a chunk longer than two pages.
C: the smallest of everything: one stream, a window of one key, a chunk of one position, one head,
one expert, a temperature that steps at every position; one layer without a mask; no value mixing.
"""
import os

ZAVESUN_A = {
    "architecture": "Zavesun", "vocab": 197, "width": 52, "norm": {"eps": 1e-5}, "streams": 3, "logit_softcap": 9.0,
    "layers": [
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 10, "vdim": 14, "scale": 0.3, "mask": {"size": 19},
                                        "q_temp": {"coef": 0.7, "every": 8}},
         "mlp": {"kind": "dense", "ff": 60}},
        {"type": "attention_2", "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 6, "scale": 0.45, "mask": {"size": 21},
                                          "rot": {"base": 100.0, "dims": 8, "scaling": {"factor": 2.5}}, "v_mix": True},
         "mlp": {"kind": "moe", "expert": {"ff": 20}, "router": {"experts": 5, "top": 2}}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.5, "mask": {"size": 7},
                                        "q_temp": {"coef": 0.3, "every": 5}, "v_mix": True},
         "mlp": None},
        {"type": "attention_2", "mixer": {"heads": 4, "kv_heads": 1, "dim": 6, "vdim": 12, "scale": 0.6, "mask": {"size": 11},
                                          "rot": {"base": 50.0, "dims": 6}, "v_mix": True},
         "mlp": {"kind": "dense", "ff": 36}},
    ],
}
ZAVESUN_B = {
    "architecture": "Zavesun", "vocab": 256, "width": 128, "norm": {"eps": 3e-6}, "streams": 2,
    "layers": [
        {"type": "attention_2", "mixer": {"heads": 4, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.18, "mask": {"size": 40},
                                          "rot": {"base": 10000.0, "dims": 32, "scaling": {"factor": 4.0}}, "v_mix": True},
         "mlp": {"kind": "moe", "expert": {"ff": 64}, "router": {"experts": 4, "top": 1}}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 4, "dim": 16, "vdim": 8, "scale": 0.25, "mask": {"size": 33},
                                        "q_temp": {"coef": 0.5, "every": 16}, "v_mix": True},
         "mlp": {"kind": "dense", "ff": 256}},
        {"type": "attention", "mixer": {"heads": 8, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.25, "mask": {"size": 48},
                                        "q_temp": {"coef": 0.2, "every": 64}, "v_mix": True},
         "mlp": {"kind": "moe", "expert": {"ff": 32}, "router": {"experts": 16, "top": 4}}},
    ],
}
ZAVESUN_C = {
    "architecture": "Zavesun", "vocab": 64, "width": 32, "norm": {"eps": 1e-6}, "streams": 1, "logit_softcap": 30.0,
    "layers": [
        {"type": "attention", "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.35, "mask": {"size": 1},
                                        "q_temp": {"coef": 1.0, "every": 1}},
         "mlp": {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 1, "top": 1}}},
        {"type": "attention_2", "mixer": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 2, "scale": 0.5, "mask": {"size": 1},
                                          "rot": {"base": 10.0, "dims": 2}},
         "mlp": {"kind": "dense", "ff": 24}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 6, "scale": 0.5},
         "mlp": None},
    ],
}
ZAVESUN = {"A": (ZAVESUN_A, 3), "B": (ZAVESUN_B, 4), "C": (ZAVESUN_C, 5)}


def write_model(cfg, folder, seed, std=0.12):
    """config.json + model.safetensors (bfloat16 matrices, short tensor names) from the engine's
    random-weights mode; the plain implementation reads the folder with its own reader."""
    from ferrum_b200.weights import write_random_model
    write_random_model(cfg, folder, seed, dtype="bfloat16", std=std)
    assert os.path.exists(os.path.join(folder, "model.safetensors"))
    return folder
