"""Writes tests/golden/reference_vectors.npz from the reference's own CPU model.

Run in a container that has the reference tree (builds oracle/_ref first):
    python tests/golden/make_golden.py
Inputs are regenerated from the seeds in `cases()` by tests/golden/cases.py; only the
reference's outputs (and a checksum of the inputs) are stored.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

import oracle  # noqa: E402
import cases  # noqa: E402


def main():
    oracle.build(with_reference=True)
    out = {}
    for name, inputs in cases.attention_cases():
        q, gate, keys, values, context = inputs
        out[f"{name}/decode"] = oracle.ref_attn_decode(q, gate, keys, values, context, cases.CAP)
        rec, split_out = oracle.ref_attn_split(q, gate, keys, values, context, cases.CAP)
        out[f"{name}/records"] = rec
        out[f"{name}/split"] = split_out
        out[f"{name}/checksum"] = cases.checksum(q, gate, keys, values)
    for name, (proj, qw, kw, position) in cases.rope_cases():
        keys = np.zeros((2, cases.CAP, 256), np.uint16)
        values = np.zeros_like(keys)
        q, gate = oracle.ref_attn_qk_rope(proj, qw, kw, keys, values, position, cases.CAP)
        out[f"{name}/q"] = q
        out[f"{name}/k"] = keys[:, position].copy()
        out[f"{name}/v"] = values[:, position].copy()
        out[f"{name}/checksum"] = cases.checksum(proj, qw, kw)
    weights, conv, state, projections = cases.gdn_chain()
    conv_w, a_log, dt_bias, norm_w = weights
    for step, proj in enumerate(projections):
        qk, v, z, conv = oracle.ref_gdn_prepare(proj, conv, conv_w)
        decay, beta = oracle.ref_gdn_gates(proj, a_log, dt_bias)
        y, state = oracle.ref_gdn_step(qk, v, decay, beta, state)
        gated = oracle.ref_gdn_gate_norm(y, z, norm_w)
        out[f"gdn/{step}/qk"] = qk
        out[f"gdn/{step}/decay"] = decay
        out[f"gdn/{step}/beta"] = beta
        out[f"gdn/{step}/y"] = y
        out[f"gdn/{step}/gated"] = gated
    out["gdn/final_conv"] = conv
    # The 2 MiB final state is stored as a per-row checksum plus one full head.
    out["gdn/final_state_head3"] = state[3].copy()
    out["gdn/final_state_rowsum"] = state.astype(np.float64).sum(axis=2)
    out["gdn/checksum"] = cases.checksum(conv_w, a_log, dt_bias, norm_w, *projections)
    for name, (x, words, scales, biases) in cases.q4_cases():
        out[f"{name}/fused"] = np.array([oracle.ref_q4_dot(x, words, scales, biases, True)], np.float32)
        out[f"{name}/separate"] = np.array([oracle.ref_q4_dot(x, words, scales, biases, False)], np.float32)
        out[f"{name}/checksum"] = cases.checksum(x, words, scales, biases)
    np.savez_compressed(os.path.join(HERE, "reference_vectors.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
