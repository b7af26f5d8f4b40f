// The CTA-pair (cta_group::2) form of the 16-bit GEMM, selected by deca_gemm_cfg.cta_group == 2.
#pragma once

#include <stdint.h>

#include "deca_b200.h"

namespace deca {

// Host-only validity of a cta_group == 2 config (BM = 128 or 256 rows per CTA, BN = 128 or 256,
// accumulators within 512 tensor-memory columns, staged epilogue, no stream-K).
int gemm16_pair_check(int64_t M, int64_t N, int64_t K, const deca_gemm_cfg *cfg);

// Launches the pair kernel; shapes, alignment and the config have been checked by the caller.
int gemm16_pair_launch(int dtype, const void *A, const void *B, void *C, int64_t M, int64_t N, int64_t K,
                       const deca_gemm_cfg *cfg, void *stream);

}  // namespace deca
