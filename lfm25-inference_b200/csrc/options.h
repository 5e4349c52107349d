// Process-wide switches of the library.  Each has a default, may be preset by an environment variable of the
// same name in upper case with the prefix LFM25_ (read once, when the first option is looked at), and can be
// changed at run time through lfm25_set_option().  The hot paths read a plain array: no getenv per launch.
//
//   name                 values                                default   meaning
//   pdl                  0 | 1                                 1         programmatic dependent launch on every kernel
//   fused_append         0 two launches | 1 one kernel | 2 auto  2       decode layers: QK-norm + RoPE + append as a kernel
//                                                                        of their own, or inside attention; auto = by
//                                                                        lfm25_decode_one_kernel_preferred()
//   fused_silu           0 | 1                                 1         E4M3 Gate/Up: SiLU(gate) * up in the GEMM epilogue
//   fused_silu_bf16      0 | 1                                 0         the same for a Gate/Up site that stays in BF16
//   kv_evict_first       0 | 1                                 1         L2 evict-first hint on the KV page stream
//   weights_evict_first  0 | 1                                 1         the same hint on the weight stream of the tcgen05 GEMMs
//   splitk_cluster_merge 0 | 1                                 1         decode executor: the KV splits of a token merge inside
//                                                                        the attention kernel (one cluster per token and KV
//                                                                        head) instead of through records and a merge kernel
//   engine_graph         0 | 1                                 1         serving engine replays captured decode steps
//   hybrid_attention     0 auto | 1 umma | 2 mma               0         kernel of the mixed-step attention
//   fp8_gemm_path        0 auto | 1 stream | 2 umma | 3 generic | 4 rows   0   kernel of the E4M3 linear
//   bf16_gemm            0 auto | 1 umma | 2 cublaslt | 3 rows  0         kernel of the BF16 linear
//   decode_splits        0 auto | 1..8                         0         KV splits of the decode attention
//   wait_limit_ns        > 0                                   1e9       limit of every bounded device-side wait
//   wait_selftest_drop   0 | 1                                 0         self-test: kernels with a TMA ring arm one
//                                                                        barrier whose copy they never issue, so that
//                                                                        the bounded wait runs out (no fault, no trap)
// Environment presets accept the numbers above; hybrid_attention, fp8_gemm_path and bf16_gemm also their names.
#pragma once

#include <stdint.h>

namespace lfm25 {

enum Option : int {
    kOptPdl = 0,
    kOptFusedAppend,
    kOptFusedSilu,
    kOptFusedSiluBf16,
    kOptKvEvictFirst,
    kOptWeightsEvictFirst,
    kOptSplitkClusterMerge,
    kOptEngineGraph,
    kOptHybridAttention,
    kOptFp8GemmPath,
    kOptBf16Gemm,
    kOptDecodeSplits,
    kOptWaitLimitNs,
    kOptWaitSelftestDrop,
    kOptCount
};

// values of fp8_gemm_path / bf16_gemm
enum GemmPath : int64_t { kPathAuto = 0, kPathStream = 1, kPathUmma = 2, kPathGeneric = 3, kPathRows = 4 };
enum Bf16Path : int64_t { kBf16Auto = 0, kBf16Umma = 1, kBf16CublasLt = 2, kBf16Rows = 3 };

// The table (defined in options.cu); initialised from the environment on first use.
int64_t option(Option which);
bool set_option_by_name(const char* name, int64_t value);
bool get_option_by_name(const char* name, int64_t* value);

inline uint64_t wait_limit_ns() { return static_cast<uint64_t>(option(kOptWaitLimitNs)); }
inline bool weights_evict_first() { return option(kOptWeightsEvictFirst) != 0; }
inline bool wait_selftest_drop() { return option(kOptWaitSelftestDrop) != 0; }

}  // namespace lfm25
