"""CPU oracle for the fused-MoE hot path.  TEST INFRASTRUCTURE, not product code.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import this package; the CUDA product path never does.  Each function is
a CPU restatement (numpy / torch on CPU tensors) of one stage of the
reference's fused-MoE path and cites the reference lines it follows
(``ref:`` = path inside the FlagGems-sglang project, ``TK:`` = the third-party
``triton_kernels`` package the reference calls into).

Pinning status
--------------
* routing metadata (``oracle.routing.standard_topk_to_routing``): PINNED against
  golden vectors produced by running the reference's own
  ``_standard_topk_to_triton_kernels`` on CPU tensors (tests/golden/).
* silu-and-mul formula and operand halves: PINNED against golden vectors made
  by running the reference's Triton kernel under the Triton interpreter.
* grouped-GEMM numerics and the end-to-end op: the arithmetic lives in the
  unpinned third-party ``triton_kernels.matmul_ogs`` and needs a GPU, so the
  end-to-end restatement is checked only against an independent dense per-token
  formulation -> "parity unpinned" for the GEMM numerics.
* router top-k, grouped top-k, moe_align_block_size, fp8 block quantisation,
  moe_sum: absent from the reference (its caller owns them) -> "parity unpinned";
  the contracts are written out in the docstrings.
"""
from . import routing, experts, quant  # noqa: F401
