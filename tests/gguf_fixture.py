"""Writes a small LLaMA-shaped GGUF file (Q4_K_M-style mix) with the third-party gguf-py writer:
quantized tensors carry the synthetic packed bytes of ``boostr_b200.synth``, so the loader's output can be
compared byte for byte with what went in."""
import numpy as np

from boostr_b200 import synth
from boostr_b200.format import QuantFormat as F

HID, KVD, FFN, VOC = 1024, 256, 2048, 1536

# gguf name -> (format, N, K)
LAYER_TENSORS = {
    "attn_q.weight": ("Q4_K", HID, HID), "attn_k.weight": ("Q4_K", KVD, HID), "attn_v.weight": ("Q6_K", KVD, HID),
    "attn_output.weight": ("Q4_K", HID, HID), "ffn_gate.weight": ("Q4_K", FFN, HID), "ffn_up.weight": ("Q8_0", FFN, HID),
    "ffn_down.weight": ("Q6_K", HID, FFN),
}


def write_gguf(path, layers=2, alignment=None):
    import gguf
    from gguf import GGMLQuantizationType as T

    qt = {"Q4_0": T.Q4_0, "Q5_0": T.Q5_0, "Q8_0": T.Q8_0, "Q2_K": T.Q2_K, "Q3_K": T.Q3_K, "Q4_K": T.Q4_K, "Q5_K": T.Q5_K, "Q6_K": T.Q6_K}
    rng = synth.rng_for(60, layers)
    w = gguf.GGUFWriter(path, "llama")
    w.add_uint32("llama.block_count", layers)
    w.add_string("general.name", "fixture")
    if alignment:
        w.add_custom_alignment(alignment)
    packed = {}

    def add(name, fmt, n, k):
        f = F.parse(fmt)
        b = synth.weight_bytes(f, rng, n, k)
        packed[name] = (fmt, n, k, b)
        w.add_tensor(name, b.reshape(n, -1), raw_dtype=qt[fmt])

    w.add_tensor("token_embd.weight", rng.standard_normal((VOC, HID), dtype=np.float32))
    for li in range(layers):
        w.add_tensor(f"blk.{li}.attn_norm.weight", rng.standard_normal(HID, dtype=np.float32))
        for suffix, (fmt, n, k) in LAYER_TENSORS.items():
            add(f"blk.{li}.{suffix}", fmt, n, k)
        w.add_tensor(f"blk.{li}.attn_q.bias", rng.standard_normal(HID, dtype=np.float32))
    w.add_tensor("output_norm.weight", rng.standard_normal(HID, dtype=np.float32).astype(np.float16))
    add("output.weight", "Q6_K", VOC, HID)
    # one tensor of every other format the library reads (expert-style names: they map to names of their own)
    for i, fmt in enumerate(("Q4_0", "Q5_0", "Q2_K", "Q3_K", "Q5_K")):
        add(f"blk.0.ffn_gate.{i}.weight", fmt, 64, HID)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return packed
