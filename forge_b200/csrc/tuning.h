/* Internal test and tuning hooks of libforge_b200.so. NOT part of the public ABI
 * (include/forge_b200.h): the symbols are exported so that the library's own tests and benchmark
 * cases can pin a kernel variant or exercise an error path, and may change without notice.
 */
#ifndef FORGE_B200_TUNING_H
#define FORGE_B200_TUNING_H

#ifdef __cplusplus
extern "C" {
#endif

/* Pin the dense tile width (64/128/256; 512 = the CTA-pair kernel) or the sparse token-tile width
 * (32/64/128; 1000 + BT = the CTA-pair kernel with BT tokens) for every later call of this
 * process; 0 restores automatic selection. Stored atomically; meant to be set between calls. */
void forge_b200_set_dense_tile(int bn);
void forge_b200_set_sparse_tile(int bt);

/* Generic integer knobs read by the kernels' launchers (key meanings are private to the
 * library's benchmark cases); unknown keys are ignored. */
void forge_b200_set_tuning(int key, int value);
int forge_b200_get_tuning(int key);

/* Copies up to 8 probe counters of the sparse CTA-pair kernel (pair-kernel flag 4) to out. */
int forge_b200_read_probe(unsigned long long* out, int n);

/* Ceiling probes (probes.cu). mma_rate: clocks per tcgen05.mma kind::i8 instruction with operands
 * resident in shared memory - pair != 0: cta_group::2 with M = 256, else M = 128; n: UMMA N (multiple
 * of 16, <= 256); sparse != 0: the 2:4 form with K = 64, else K = 32; commits: tcgen05.commit per four
 * instructions (0, 1 or 2); ctas: CTAs launched (all time themselves, CTA 0 reports). tma_ingest: mean
 * bytes per clock and CTA when `ctas` CTAs stream 128 x 128-byte tiles of `matrix` (rows x kcols int8)
 * with `producers` TMA-issuing threads each. Both synchronise the device and return a negative status
 * code on failure. */
double forge_b200_probe_mma_rate(int pair, int n, int sparse, int commits, int ctas);
double forge_b200_probe_tma_ingest(const void* matrix, int rows, int kcols, int producers, int ctas);

/* Launches one thread block that waits, for at most budget_us microseconds (clamped to
 * 10000), on a barrier nobody arrives at - the way every bounded wait of the GEMM kernels gives
 * up - and then records raw code 900 in the device status word and returns normally. */
int forge_b200_selftest_wait_timeout(unsigned budget_us, void* stream);

#ifdef __cplusplus
}
#endif

#endif
