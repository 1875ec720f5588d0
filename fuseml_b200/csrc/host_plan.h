// Internal declarations shared by the host-only planner and the CUDA launch file.
#pragma once

#include <stdint.h>

#include "../../include/fuseml_sm100.h"

namespace fuseml {

int dtype_bytes(int32_t dt);
void default_props(fuseml_device_props_t* p);
int validate_desc(const fuseml_gemm_desc_t* d);
// `allow_split_k = false` keeps the workspace free of partial tiles (fixed-budget callers).
int make_plan(const fuseml_gemm_desc_t* d, const fuseml_device_props_t* props, fuseml_plan_t* plan,
              bool allow_split_k = true);

// How B sits in memory: 0 = K contiguous (nn.Linear weight view), 1 = N
// contiguous (row-major [K,N]), -1 = neither can be described by a TMA map.
int b_layout(const fuseml_gemm_desc_t* d);
// How A sits in memory: 0 = K contiguous, 1 = M contiguous (stored [K,M]), -1 = not addressable.
int a_layout(const fuseml_gemm_desc_t* d);

// Leading dimension (elements) of the [rows, 3K] hi|lo|hi split copies that
// fp32 operands are expanded into before the TF32 MMA.
int64_t split_ld(int64_t K);

struct WorkspaceLayout {
  int64_t split_a_off, split_b_off;  // fp32 operands only
  int64_t red_sum_off, red_max_off;  // reduction partials
  int64_t partials, len;             // partial arrays are [partials][len]
  int64_t splitk_off;                // split-K: fp32 partial tiles, [split_k][tiles][128 x tile_n]
  int64_t sk_ws_off, sk_flags_off;   // stream-K: one partial slot (128 x 256 fp32) and one flag per CTA
  int64_t sk_flags_bytes;
  int64_t total;
};
void workspace_layout(const fuseml_gemm_desc_t* d, const fuseml_plan_t* plan, WorkspaceLayout* w);

}  // namespace fuseml
