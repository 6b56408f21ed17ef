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

/* A device buffer of 8 x 256 int64 that the MMA issuer of CTA pair 0 of the 256 x 384 kernel fills, per tile, with
 * SM-clock stamps and the cycles it spent in each kind of wait (tile start, after the accumulator waits, cycles
 * waiting for operands / scales / the second accumulator, tile end, wait for the first operands); null switches the
 * stamping off (the default). */
int smoe_internal_gemm_trace(void* device_buffer);

#ifdef __cplusplus
}
#endif
#endif /* SMOE_INTERNAL_H_ */
