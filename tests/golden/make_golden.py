"""Generate the golden fixtures in this directory from the REAL reference code.

Run once, in a container that has the reference checkout and a copy of the
third-party ``triton_kernels`` package (vLLM vendors one):

    python tests/golden/make_golden.py --reference <checkout>/src \
        --triton-kernels <site-packages>/vllm/third_party

The tests only read the ``.npz`` files written here; they never import the
reference.  What is captured:

* ``routing_*.npz``: output of the reference's own
  ``flaggems_sglang.ops.fused_moe._standard_topk_to_triton_kernels`` on CPU
  tensors, for the reference's test shapes and seeds
  (tests/test_fused_moe.py:64-72, tests/accuracy_utils.py:112-139) plus two
  skewed cases with empty experts.
* ``silu_*.npz``: the reference's Triton ``_silu_and_mul_kernel`` /
  ``_silu_and_mul_sigmoid_kernel`` run under the Triton interpreter
  (TRITON_INTERPRET=1) with an fp32 output buffer, so the stored values are the
  fp32 results before any output rounding (the interpreter truncates instead of
  rounding when it stores into bf16, so a bf16 output would not be faithful).
* ``swiglu_*.npz``: ``triton_kernels.swiglu.swiglu_torch`` (the third-party library's torch reference of the
  gated unit the reference's bias variant names) on seeded fp32 inputs, with and without the clamp.
"""
import argparse
import os
import sys
import tempfile

import numpy as np


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--triton-kernels", required=True)
    args = ap.parse_args()

    os.environ["DNN_VENDOR"] = "nvidia"
    os.environ["TRITON_INTERPRET"] = "1"
    stub = tempfile.mkdtemp()
    os.makedirs(os.path.join(stub, "sgl_kernel"))
    with open(os.path.join(stub, "sgl_kernel", "__init__.py"), "w") as f:
        f.write("def gelu_and_mul(x, out):\n    raise NotImplementedError\n")
    sys.path[:0] = [args.reference, args.triton_kernels, stub]

    import torch
    import flaggems_sglang  # noqa: F401
    from flaggems_sglang.ops import fused_moe as fm

    here = os.path.dirname(os.path.abspath(__file__))

    # ---- routing ---------------------------------------------------------
    shapes = [
        (1, 128, 256, 8, 2), (7, 128, 256, 8, 2), (33, 256, 512, 16, 4),
        (1, 1280, 3072, 64, 8), (4, 1280, 3072, 64, 8), (17, 1280, 3072, 64, 8),
        (64, 1280, 3072, 64, 8), (1024, 1280, 3072, 64, 8),
    ]
    cases = []
    for (M, K, N, E, topk) in shapes:
        torch.manual_seed(M + K + N + E + topk)
        logits = torch.randn(M, E, dtype=torch.float32)
        cases.append((f"M{M}_E{E}_k{topk}", logits, topk, E))
    g = torch.Generator().manual_seed(1234)
    for (T, E, topk) in [(40, 32, 4), (256, 128, 8)]:
        logits = torch.randn(T, E, generator=g)
        logits[:, : E // 2] -= 30.0  # half of the experts never selected
        logits[:, E // 2] += 4.0  # one hot expert
        cases.append((f"skew_T{T}_E{E}_k{topk}", logits, topk, E))

    for name, logits, topk, E in cases:
        w = torch.softmax(logits, dim=-1)
        tw, ti = torch.topk(w, k=topk, dim=-1)
        tw = tw / tw.sum(dim=-1, keepdim=True)
        rd, gi, si = fm._standard_topk_to_triton_kernels(tw, ti, E)
        ed = rd.expt_data
        out = dict(
            logits=logits.numpy(), topk_weights=tw.numpy(), topk_ids=ti.numpy().astype(np.int32),
            gate_scal=rd.gate_scal.numpy(), hist=rd.expt_hist.numpy(),
            topk_indx=gi.src_indx.numpy(), gate_indx=gi.dst_indx.numpy(),
            scatter_src=si.src_indx.numpy(), scatter_dst=si.dst_indx.numpy(),
            token_offs_raw=ed.token_offs_raw.numpy(),
        )
        for bm in (16, 32, 64, 128):
            out[f"token_offs_pad_{bm}"] = ed.token_offs_pad[bm].numpy()
            out[f"block_pid_map_{bm}"] = ed.block_pid_map[bm].numpy()
        np.savez_compressed(os.path.join(here, f"routing_{name}.npz"), **out)
        print("wrote routing", name)

    # ---- silu-and-mul (both row-count branches: rows<=128 and rows>128) ----
    g = torch.Generator().manual_seed(7)
    for rows, half in [(5, 96), (130, 40)]:
        y1 = (torch.randn(rows, 2 * half, generator=g) * 3.0).to(torch.bfloat16)
        out = torch.empty(rows, half, dtype=torch.float32)
        fm._silu_and_mul_triton(y1, out)
        np.savez_compressed(
            os.path.join(here, f"silu_rows{rows}_half{half}.npz"),
            y1_bits=y1.view(torch.int16).numpy(), out_f32=out.numpy(),
        )
        print("wrote silu", rows, half)

    # ---- swiglu of the bias variant: the third-party library's own torch reference ----
    # (the reference op only names `swiglu_fn`, src/flaggems_sglang/ops/fused_moe.py:261; the arithmetic is
    # triton_kernels.swiglu, vendored copy given by --triton-kernels)
    from triton_kernels.swiglu import PrecisionConfig as SwigluPrecisionConfig
    from triton_kernels.swiglu import swiglu_torch

    for rows, half, alpha, limit in [(9, 64, 1.702, 7.0), (33, 40, 1.0, None), (4, 128, 1.702, 0.75)]:
        a = torch.randn(rows, 2 * half, generator=g) * 4.0
        out = swiglu_torch(a, alpha, SwigluPrecisionConfig(limit=limit))
        np.savez_compressed(
            os.path.join(here, f"swiglu_rows{rows}_half{half}.npz"),
            a_f32=a.numpy(), out_f32=out.numpy(), alpha=np.float32(alpha),
            limit=np.float32(-1.0 if limit is None else limit),
        )
        print("wrote swiglu", rows, half)


if __name__ == "__main__":
    main()
