/* novadit_b200_tuning.h - tuning and diagnostic hooks of libnovadit_b200.so.
 *
 * Not part of the operator interface (novadit_b200.h): these are the switches the benchmark sweeps and the
 * timeline scripts use to force a kernel variant or to collect device-side timestamps. They are process-wide
 * atomics read at launch time; a program that flips one while another thread launches gets either setting.
 * The operator entry points are re-entrant as long as nobody calls these. None has a counterpart in the
 * reference.
 */
#ifndef NOVADIT_B200_TUNING_H_
#define NOVADIT_B200_TUNING_H_

#ifdef __cplusplus
extern "C" {
#endif

/* Tuning hook: force the row-tile height of the generic norm kernels (0 = built-in choice).
 * Process-wide; affects nd_norm_dparam_ws_bytes. No counterpart in the reference. */
void nd_tune_norm_tile_rows(int tile_rows);
/* Tuning hook: 0 = default, 1 = generic kernels for every shape, 3 / 4 = never / always run the forward pass
 * with the chunked warp-per-row kernel where it applies, 5 = even row chunks instead of sample-aligned ones, 6 =
 * the general bulk-copy backward kernel also where the flat walk applies.
 * Results are identical up to fp32 summation order. */
void nd_tune_norm_variant(int variant);
/* Tuning hook: pipeline depth (shared-memory stages) of the bulk-copy norm kernels; 0 = as many as
 * fit the per-CTA budget. No counterpart in the reference. */
void nd_tune_norm_stages(int stages);
/* Tuning hook: 0 launches the norm kernels without programmatic stream serialization (default 1:
 * each kernel may be scheduled while its predecessor in the stream drains). */
void nd_tune_norm_pdl(int enabled);
/* Tuning hook: cap on CTAs per SM of the bulk-copy norm kernels (0 = what occupancy allows). */
void nd_tune_norm_chunks_per_sm(int n);
/* Test hook for the abort path of the bulk-copy norm kernels. `limit_ns` bounds every wait on a bulk copy (0
 * restores the default of one second); with `withhold_first_copy` != 0 CTA 0 never sends its first copy, so its
 * first wait expires with nothing in flight: the kernel sets the device error word (nd_device_error: 1 forward,
 * 2 backward), the CTA leaves through the abort path and the launch completes; the context stays usable and the
 * launch's output is incomplete. Process-wide; tests reset both. */
void nd_tune_norm_wait_test(unsigned long long limit_ns, int withhold_first_copy);
/* Tuning hook for the gate-act kernels: rows per CTA group (1, 2 or 4; 0 = default) and 1 = a single
 * resident wave of CTAs striding over the groups instead of one CTA per group (default 0). Process-wide.
 * No counterpart in the reference. */
void nd_tune_gate_act(int rows_per_group, int persistent);
/* Tuning hook: 1 = two-CTA tiles (tcgen05 cta_group::2 over clusters of two CTAs), 0 = single-CTA
 * tiles, negative (default) = chosen per problem. Process-wide. No counterpart in the reference. */
void nd_tune_fc1_pair(int mode);
/* Tuning hook: 0 launches the FC1 kernels without programmatic stream serialization (default 1: barrier set-up,
 * tensor-memory allocation and tensor-map prefetch of a launch may run while its predecessor in the stream drains;
 * every kernel executes griddepcontrol.wait before its first global access). The CTA-pair backward GEMM, whose
 * predecessor in the stream is a memset, is always launched without. */
void nd_tune_fc1_pdl(int enabled);
/* The same choice for the backward GEMMs (nd_fc1_bwd_gemm) when a workspace is given: 1 = 256 x 256 tiles over CTA
 * pairs with the k-blocks shared out evenly, 0 = whole 128 x 192 single-CTA tiles, negative (default) = chosen per
 * problem. Process-wide. No counterpart in the reference. */
void nd_tune_fc1_bwd_pair(int mode);
/* Diagnostic hook: a device array of 8 int64 that later nd_fc1_fwd launches add cycle counters to
 * ([0] copy thread waiting for a free stage, [3]/[4] one epilogue warp waiting / working, [5]/[7] the
 * copy thread's lifetime in cycles / nanoseconds); NULL (default) turns it off. The CTA-pair launches of
 * nd_fc1_bwd_gemm add, per cluster, the issuing thread's [0] cycles waiting for a drained accumulator, [1]
 * cycles waiting for operands, [5] lifetime in cycles, [6] one, [7] its number of k-blocks. No counterpart in
 * the reference. */
void nd_tune_fc1_trace(long long* device_counters);

#ifdef __cplusplus
}
#endif
#endif /* NOVADIT_B200_TUNING_H_ */
