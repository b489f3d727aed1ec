#!/usr/bin/env python3
"""Makes tests/golden/reference_tiny_a.npz: logits of the reference's OWN engine on a tiny model.

The reference's LFM2 model code is CUDA (``libgpu_engine.so``); it cannot run on a CPU, so this
script runs on a machine with a GPU, once:

    baseline/build_reference.sh                      # the reference's library, unmodified
    python tests/golden/make_reference_golden.py     # writes tests/golden/reference_tiny_a.npz

It writes the Tiny A model folder (``write_random_model(TINY_A, seed 0)``: the reference's
engine rotates adjacent pairs, as Tiny A does, and needs heads * head_dim == hidden, as Tiny A
has), loads those weights into the reference through its stock entry points
(baseline/reference_arm.py), prefills a prompt (cuda_prefill_batch), then feeds given tokens one
by one (cuda_decode_step_gpu) and keeps the float32 logits its LM head returns after the prompt
and after every fed token.  ``tests/test_golden_reference.py`` compares the plain implementation
with these numbers on the CPU.
"""
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path[:0] = [ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "baseline")]

PROMPT_LEN, FED = 41, 30
SEED_MODEL, SEED_TOKENS = 0, 123


def read_bf16_safetensors(path):
    """name -> float32 array of a safetensors file whose tensors are BF16 (no torch in this process:
    the reference's library brings the CUDA toolkit's runtime, torch would bring its own)."""
    import json
    import struct
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        assert e["dtype"] == "BF16", (name, e["dtype"])
        lo, hi = e["data_offsets"]
        bits = np.frombuffer(data[lo:hi], dtype="<u2").astype(np.uint32) << 16
        out[name] = bits.view(np.float32).reshape(e["shape"])
    return out


def main():
    import subprocess
    from tiny_configs import TINY_A
    import reference_arm

    cfg = dict(TINY_A)
    with tempfile.TemporaryDirectory() as d:
        subprocess.run([sys.executable, "-c",
                        "import sys; sys.path[:0] = %r; from tiny_configs import TINY_A; "
                        "from neurogrid_b200.weights import write_random_model; write_random_model(TINY_A, %d, %r)"
                        % ([ROOT, os.path.join(ROOT, "tests")], SEED_MODEL, d)], check=True)
        tensors = read_bf16_safetensors(os.path.join(d, "model.safetensors"))
    checksum = float(sum(np.abs(v).astype(np.float64).sum() for v in tensors.values()))
    ref_cfg = dict(cfg, head_dim=cfg["hidden_size"] // cfg["num_attention_heads"], intermediate_size=192)
    ref = reference_arm.Reference(ref_cfg, max_batch=1, tensors=tensors)
    tokens = np.random.default_rng(SEED_TOKENS).integers(0, cfg["vocab_size"], PROMPT_LEN + FED).tolist()
    rows = []
    ref.prefill(0, tokens[:PROMPT_LEN])
    ref.restore_states(0)
    ref._h2d(ref.block_table_gpu, ref.tables[0])
    ref.first_token(0)
    rows.append(ref.logits_to_host().copy())                 # logits at the prompt's last position
    for t in tokens[PROMPT_LEN:]:
        ref.decode_one(0, t, stock=True)
        rows.append(ref.logits_host.copy())                  # logits at the fed token's position
    ref.sync()
    out = os.path.join(HERE, "reference_tiny_a.npz")
    np.savez_compressed(out, tokens=np.asarray(tokens, dtype=np.int32), logits=np.stack(rows).astype(np.float32),
                        prompt_len=PROMPT_LEN, seed_model=SEED_MODEL, weights_abs_sum=checksum)
    print("wrote", out, np.stack(rows).shape, "max |logit|", float(np.abs(np.stack(rows)).max()))


if __name__ == "__main__":
    main()
