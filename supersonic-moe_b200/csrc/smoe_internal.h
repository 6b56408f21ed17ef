/* Symbols the library exports for its own tests and timing experiments.  They are NOT part of the product ABI
 * (include/smoe_b200.h): process-global, unsynchronised, and able to switch stores off. */
#ifndef SMOE_INTERNAL_H_
#define SMOE_INTERNAL_H_

#ifdef __cplusplus
extern "C" {
#endif

/* bits 0..15: force the GEMM column tile (128, 192 or 256; 0 = automatic); bit 16: epilogues skip their stores;
 * bit 17: force the single-CTA kernel; bit 18: the fused dgated epilogue is skipped whole;
 * bits 19..23: timing experiments of the two-CTA main loop (no operand loads after the first ring pass,
 * no accumulator drain, no scale copies, ...).  0 restores the defaults. */
int smoe_internal_gemm_knobs(int bits);

#ifdef __cplusplus
}
#endif
#endif /* SMOE_INTERNAL_H_ */
