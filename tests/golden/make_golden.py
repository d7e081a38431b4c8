"""Generate the golden vectors under tests/golden/ from the REFERENCE's own code.

Run in the authoring container only (needs the reference checkout, which is
not present where the GPU tests run):

    python tests/golden/make_golden.py /path/to/PaddlePaddle-FlashMask

It imports the reference's mask generators and bias expander
(tests/common/startend_row_indices.py) and its eager fp32 attention
(tests/torch/attention_ref.py, differentiated with torch.autograd as the
reference's own tests do, tests/torch/test_flashmask.py:261-319) and stores
inputs and outputs as ``attention_<case>.npz``.  ``attention_ref(causal=True)``
builds its triangle on "cuda" (attention_ref.py:19-20); on the CPU the
triangle comes from the bias expander instead (startend_row_indices.py:211-214),
which is the same mathematics.
"""
import importlib.util
import os
import sys
import zlib

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from flashmask_b200 import workloads as W  # noqa: E402


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(ref_root):
    gen = _load(os.path.join(ref_root, "tests/common/startend_row_indices.py"), "ref_masks")
    ref = _load(os.path.join(ref_root, "tests/torch/attention_ref.py"), "ref_attention")

    S = 64
    rng = np.random.default_rng(2026)
    docs3 = [20, 14, 30]
    cases = []
    # (name, idx, causal, Sq, Sk, sink?)  — reference generators first
    cases.append(("none_causal", None, True, S, S, False))
    cases.append(("none_full", None, False, S, S, True))
    cases.append(("ref_non_causal",) + gen.non_causal_mask(1, S, S, 1) + (S, S, False))
    cases.append(("ref_causal",) + gen.causal_mask(1, S, S, 1) + (S, S, False))
    cases.append(("ref_sliding_window",) + gen.sliding_window_mask(1, S, S, 1, window_size=9) + (S, S, True))
    cases.append(("ref_causal_document",) + gen.causal_document_mask(1, S, S, 1, doc_seqlens=list(docs3)) + (S, S, False))
    cases.append(("ref_document",) + gen.document_mask(1, S, S, 1, doc_seqlens=list(docs3)) + (S, S, True))
    cases.append(("ref_prefix_lm_document",) + gen.prefix_lm_document_mask(
        1, S, S, 1, doc_seqlens=[(8, 20), (14, 14), (4, 30)]) + (S, S, False))
    cases.append(("ref_prefix_lm_causal",) + gen.prefix_lm_causal_mask(1, S, S, 1, prefix_length=10) + (S, S, False))
    # rectangular (Sq != Sk): bottom-right aligned causal triangle
    cases.append(("ref_causal_document_rect",) + gen.causal_document_mask(
        1, 48, 80, 1, doc_seqlens=[30, 20, 30]) + (48, 80, False))
    # generators of this repository, expanded by the reference's bias expander
    cases.append(("share_question",) + W.share_question(1, S, S, 16, 8, 2) + (S, S, False))
    cases.append(("random_eviction",) + W.random_eviction(1, S, S, rng) + (S, S, True))
    cases.append(("four_column",) + W.four_column_bands(1, S, S, rng) + (S, S, False))
    cases.append(("empty",) + W.empty_mask(1, S, S) + (S, S, True))

    Hq, Hkv, d, dv = 2, 1, 16, 16
    for name, idx, causal, Sq, Sk, use_sink in cases:
        g = torch.Generator().manual_seed(zlib.crc32(name.encode()))
        q = torch.randn(1, Sq, Hq, d, generator=g, requires_grad=True)
        k = torch.randn(1, Sk, Hkv, d, generator=g, requires_grad=True)
        v = torch.randn(1, Sk, Hkv, dv, generator=g, requires_grad=True)
        do = torch.randn(1, Sq, Hq, dv, generator=g)
        sink = torch.randn(Hq, generator=g, requires_grad=True) if use_sink else None
        if idx is None:
            bias_np = gen.startend_row_indices_to_attn_bias(
                np.full((1, 1, Sk, 1), Sq, dtype=np.int32), Sq, Hq, causal=True) if causal else None
        else:
            bias_np = gen.startend_row_indices_to_attn_bias(np.asarray(idx), Sq, Hq, causal=causal)
        bias = None if bias_np is None else torch.from_numpy(bias_np)
        out, _ = ref.attention_ref(q, k, v, attn_bias=bias, causal=False, learnable_sink=sink)
        grads = torch.autograd.grad(out, [q, k, v] + ([sink] if use_sink else []), do)
        blob = dict(q=q.detach().numpy(), k=k.detach().numpy(), v=v.detach().numpy(),
                    do=do.numpy(), out=out.detach().numpy(), dq=grads[0].numpy(),
                    dk=grads[1].numpy(), dv=grads[2].numpy(), causal=np.int32(causal),
                    Sq=np.int32(Sq), Sk=np.int32(Sk))
        if idx is not None:
            blob["idx"] = np.asarray(idx, dtype=np.int32)
        if use_sink:
            blob["sink"] = sink.detach().numpy()
            blob["dsink"] = grads[3].numpy()
        if bias_np is not None:
            blob["visible"] = np.packbits(np.isfinite(bias_np[:, :1]).reshape(-1))
        np.savez_compressed(os.path.join(HERE, f"attention_{name}.npz"), **blob)
        print("wrote", name, "out|max|", float(out.detach().abs().max()))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
