"""Generate the end-to-end fixtures ``e2e_*.npz`` from the REAL reference operator, on a GPU.

Run once on a machine with a CUDA device, an installed copy of the reference package and a copy of the
third-party ``triton_kernels`` package (vLLM vendors one):

    python tests/golden/make_golden_e2e.py --reference <dir that holds flaggems_sglang/> \
        [--triton-kernels <site-packages>/vllm/third_party] [--out tests/golden]

Every case calls ``flaggems_sglang.triton_kernel_fused_experts``
(src/flaggems_sglang/ops/fused_moe.py:149-232) with routing tables made by the reference's own
``_standard_topk_to_triton_kernels`` (:119-146) and stores what the operator returned.  Shapes and seeds are
the reference's test list (tests/test_fused_moe.py:64-72, tests/accuracy_utils.py:112-139): the three small
shapes and M in {1, 4, 17, 64, 1024} at K=1280, N=3072, E=64, top-k 8, with both values of
``apply_router_weight_on_input``.  (``scatter_indx=None`` is not captured: the reference operator itself raises
for it whenever top-k > 1, because it ends with ``output.view(num_tokens, hidden_size)``, fused_moe.py:232.)  Inputs come from a counter-based generator (``e2e_inputs`` in tests/util.py) that gives the same
values on the CPU and on a GPU, so that the tests regenerate them instead of storing a gigabyte of weights;
per-expert checksums of every input tensor are stored and compared before a fixture is used.

The tests only read the ``.npz`` files; they never import the reference.
"""
import argparse
import os
import sys
import tempfile

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from tests.util import checksum, e2e_inputs, stored_rows  # noqa: E402  (shared with the tests that read the fixtures)

SMALL = [(1, 128, 256, 8, 2), (7, 128, 256, 8, 2), (33, 256, 512, 16, 4)]
LARGE = [(1, 1280, 3072, 64, 8), (4, 1280, 3072, 64, 8), (17, 1280, 3072, 64, 8), (64, 1280, 3072, 64, 8),
         (1024, 1280, 3072, 64, 8)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--triton-kernels", default=None)
    ap.add_argument("--out", default=os.path.dirname(os.path.abspath(__file__)))
    args = ap.parse_args()

    os.environ["DNN_VENDOR"] = "nvidia"
    stub = tempfile.mkdtemp()
    os.makedirs(os.path.join(stub, "sgl_kernel"))
    with open(os.path.join(stub, "sgl_kernel", "__init__.py"), "w") as f:
        f.write("def gelu_and_mul(x, out):\n    raise NotImplementedError\n")
    tk = args.triton_kernels
    if tk is None:
        import vllm

        tk = os.path.join(os.path.dirname(vllm.__file__), "third_party")
    sys.path[:0] = [args.reference, tk, stub]

    import flaggems_sglang
    from flaggems_sglang.ops import fused_moe as fm

    assert torch.cuda.is_available(), "the reference operator needs a CUDA device"
    dev = torch.device("cuda", 0)
    os.makedirs(args.out, exist_ok=True)

    for shape in SMALL + LARGE:
        M, K, N, E, topk = shape
        xd, w1d, w2d, logits = e2e_inputs(*shape, device=dev)
        hidden, w1, w2 = xd, w1d, w2d
        p = torch.softmax(logits, dim=-1)
        tw, ti = torch.topk(p, k=topk, dim=-1)
        tw = tw / tw.sum(dim=-1, keepdim=True)
        rd, gi, si = fm._standard_topk_to_triton_kernels(tw, ti, E)
        out = dict(shape=np.array(shape, dtype=np.int64), topk_weights=tw.cpu().numpy(),
                   topk_ids=ti.cpu().numpy().astype(np.int32),
                   sum_hidden=checksum(hidden), sum_w1=checksum(w1), sum_w2=checksum(w2), sum_logits=checksum(logits))
        small = shape in SMALL
        variants = [("out", False)]
        if small or M <= 64:
            variants.append(("out_on_input", True))
        for key, on_input in variants:
            res = flaggems_sglang.triton_kernel_fused_experts(xd, w1d, w2d, rd, gi, si, apply_router_weight_on_input=on_input)
            torch.cuda.synchronize()
            res = res.reshape(-1, K).cpu()
            rows = stored_rows(res.shape[0])
            out[key + "_rows"] = rows
            out[key + "_bits"] = res[torch.from_numpy(rows)].contiguous().view(torch.int16).numpy()
            out[key + "_n"] = np.int64(res.shape[0])
        name = f"e2e_M{M}_K{K}_N{N}_E{E}_k{topk}.npz"
        np.savez_compressed(os.path.join(args.out, name), **out)
        print("wrote", name, {k: v.shape for k, v in out.items() if k.endswith("_bits")}, flush=True)


if __name__ == "__main__":
    main()
