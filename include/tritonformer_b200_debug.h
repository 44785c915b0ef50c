/*
 * tritonformer_b200 -- test and tuning switches of the kernel library.  Not part of the operator
 * interface: nothing here has a counterpart in the reference, and a host that only runs the
 * operators never needs this file.
 */
#ifndef TRITONFORMER_B200_DEBUG_H
#define TRITONFORMER_B200_DEBUG_H

#ifdef __cplusplus
extern "C" {
#endif

/* Test and tuning switches.
 *   key 0: value 1 sends every GEMM to the generic-stride kernel.
 *   key 1: value 1 sends every attention call to the mma.sync kernels.
 *   key 2: attention: bit 0 skips the dQ accumulation, bit 1 turns the cycle counters on, bit 5 (32) walks the
 *          (tile, batch*head) items slice by slice instead of longest first, bit 6 (64) adds dQ with vector
 *          atomics instead of the TMA reduction, bit 7 (128) keeps only the barriers of the backward's compute
 *          warps going (timing experiments: results are then meaningless).
 *   key 3: value 1 launches every kernel fully serialised (no programmatic dependent launch: a
 *          kernel's set-up no longer overlaps its predecessor's tail).
 *   key 4: GEMM: bit 0 whole tiles only (no sharing of a tile's contraction between SMs), bit 5 (32)
 *          no CTA-pair kernel, bit 6 (64) per-CTA timeline counters of the CTA-pair kernel.
 *   key 5: which counters tfb_debug_counters returns: -1 attention backward, -3 attention forward,
 *          n >= 0 the CTA-pair GEMM timeline of CTA n.
 *   key 6: how many SMs the persistent GEMM grids leave free (for a collective that runs beside
 *          them on another stream); 0 by default.                                */
void tfb_debug_set(int key, int value);
/* Timing counters of the attention backward kernel (16 cycle sums, filled while tfb_debug_set(2, 2)
 * is in effect); copies and clears them.  Synchronises the device.                        */
int tfb_debug_counters(unsigned long long* out16);

/* Launches a one-warp kernel that takes tensor memory, waits `limit_ns` nanoseconds on an mbarrier
 * that nothing arrives at, gives up, records 0x7e00 in the device status word, frees its tensor memory
 * and returns: the expiry path of the library's bounded waits, without a fault, a trap or an unbounded
 * spin.  waited_ok (device int, may be null) receives 0 when the wait ran out.  Tests only.        */
int tfb_debug_wait_probe(unsigned long long limit_ns, int* waited_ok, void* stream);

#ifdef __cplusplus
}
#endif
#endif
