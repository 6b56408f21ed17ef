/* Symbols the library exports for its own tests and timing experiments.  They are NOT part of the product ABI
 * (include/smoe_b200.h): process-global, unsynchronised, and able to switch stores off. */
#ifndef SMOE_INTERNAL_H_
#define SMOE_INTERNAL_H_

#ifdef __cplusplus
extern "C" {
#endif

/* bits 0..15: force the GEMM column tile (128, 192, 256 or 384; 0 = automatic); bit 16: epilogues skip their stores;
 * bit 17: force the single-CTA kernel; bit 18: the fused dgated epilogue is skipped whole;
 * timing experiments of the two-CTA main loops: bit 19: no operand loads after the first ring pass; bit 20: the
 * accumulators are handed back undrained (and nothing is stored); bit 21: no scale copies into TMEM;
 * bits 24..25: ring stages left unused; bits 26..30: value + 1 of the L2 prefetch distance (256-wide kernels) or of
 * the head / tail length (256 x 384 kernel), 0 = the kernel's default; bit 31: indexed A rows through TMA gather4
 * instead of the cp.async load warps.  0 restores the defaults. */
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
