"""CPU oracle for the integer-only W8A8 forward path (TEST INFRASTRUCTURE ONLY).

Everything under this package is a checker: a numpy / plain-C restatement of the
reference's arithmetic for each op on the path.  Only the test-suite, the smoke
check and the CPU-baseline leg of the benchmark may import it.  The product
package never does; its entry points fail loudly when the CUDA library is absent.

Parity status of each restatement (pinned = verified bit-for-bit against the
reference's own Python implementation run on CPU, via the committed fixtures in
``tests/golden``; unpinned = the reference has no integer implementation of that
step, the restatement is the definition):

  fixed_point.to_fixed / from_fixed            pinned
  fixed_point.rmsnorm_v2 / fused_add_rmsnorm_v2 pinned (Triton interpreter runs)
  fixed_point.silu_and_mul                     pinned (Triton interpreter runs)
  fixed_point.fwht_q15 / blockwise_fwht_q15    pinned
  fixed_point.rope_q15 / rope_fwht_q15         pinned
  fixed_point.per_token_quant_from_q15         pinned
  attention.context_attention (per-tensor)     pinned
  attention.paged_attention (per-key scales)   parity unpinned; reduces to the
                                               pinned function for uniform scales
  linear.int32_accumulate                      exact by arithmetic
  linear.requant_q15 / absmax_to_mul_shift     parity unpinned (the reference's
                                               epilogue is a float library call)
"""
