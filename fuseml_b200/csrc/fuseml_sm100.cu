// C ABI of the sm_100a backend: tensor-map construction, kernel selection and
// launch.  Everything here enqueues work on the caller's stream and returns;
// no device memory is allocated or freed.

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <atomic>
#include <cstring>
#include <initializer_list>
#include <mutex>

#include "../../include/fuseml_sm100.h"
#include "aux_kernels.cuh"
#include "gemm_kernel_v2.cuh"
#include "mlp_small_kernel.cuh"
#include "splitk_finish.cuh"
#include "host_plan.h"

namespace fuseml {

// Status word written by bounded waits that ran out (0 = none did).
__device__ int32_t g_status_word = 0;

// Diagnostics copied into every launch's parameters (fuseml_sm100_set_diagnostics).
static std::atomic<uint32_t> g_diag_wait_limit_us{0};
static std::atomic<int32_t> g_diag_drop_last_load{0};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

// 2-D row-major view [rows, cols] with `ld` elements between rows; box = {box_cols, box_rows},
// 128-byte swizzle (box_cols * element size == 128).
static int encode_2d(CUtensorMap* tm, int32_t dtype, const void* base, int64_t rows, int64_t cols, int64_t ld,
                     uint32_t box_cols, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return FUSEML_E_DEVICE;
  const int eb = dtype_bytes(dtype);
  CUtensorMapDataType dt = dtype == FUSEML_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                         : dtype == FUSEML_F16  ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  // a single row needs no real stride, but the encoder still wants a multiple of 16 bytes
  int64_t stride_bytes = ld * eb;
  if (rows == 1) stride_bytes = ((cols * eb + 15) / 16) * 16;
  cuuint64_t gstride[1] = {static_cast<cuuint64_t>(stride_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(tm, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FUSEML_OK : FUSEML_E_LAYOUT;
}

constexpr int kMaxDevices = 64;

// Per kernel instantiation and per device: the opt-in shared-memory attribute (sticky per
// device function) and, for CTA pairs, how many clusters the device holds at once.  Looked up
// once per device under a lock, so host threads driving different GPUs do not race; the
// library has to be reloaded after cudaDeviceReset (the cached state describes the old context).
struct InstanceState {
  std::mutex mutex;
  bool configured[kMaxDevices] = {false};
  int max_clusters[kMaxDevices] = {0};
};

template <int BN, int STAGES, int LAYOUT, int PROG, int CG, int EW>
static int launch_instance(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tr, const CUtensorMap& td,
                           const GemmParams& p, int grid, cudaStream_t stream) {
  using L = v2::Smem<BN, STAGES, CG>;
  auto kernel = v2::gemm_epilogue_kernel_v2<BN, STAGES, LAYOUT, PROG, CG, EW>;
  static InstanceState state;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return FUSEML_E_DEVICE; }
  int max_clusters = 0;
  {
    std::lock_guard<std::mutex> lock(state.mutex);
    if (!state.configured[dev]) {
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes) != cudaSuccess) {
        cudaGetLastError();
        return FUSEML_E_LAUNCH;
      }
      int n = 0;
      if (CG == 2) {
        // how many CTA pairs the device can hold at once (GPCs with an odd SM count lose one SM)
        cudaLaunchConfig_t q = {};
        q.gridDim = dim3(2 * 148);
        q.blockDim = dim3(v2::threads_for(EW));
        q.dynamicSmemBytes = L::kDynamicBytes;
        cudaLaunchAttribute qa[1];
        qa[0].id = cudaLaunchAttributeClusterDimension;
        qa[0].val.clusterDim.x = 2; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
        q.attrs = qa; q.numAttrs = 1;
        if (cudaOccupancyMaxActiveClusters(&n, kernel, &q) != cudaSuccess || n <= 0) { cudaGetLastError(); n = 0; }
      }
      state.max_clusters[dev] = n;
      state.configured[dev] = true;
    }
    max_clusters = state.max_clusters[dev];
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  // K-split last wave: CTA pairs wait for other pairs of the same launch, so all of them have to
  // be resident at once.  Alone on the device they are (the grid is clamped to what the device
  // holds), but next to another persistent kernel on another stream each could hold SMs the other
  // is waiting for.  A cooperative launch starts only when the whole grid fits, which rules that
  // out; it replaces the programmatic dependent launch for these (long) kernels (both attributes
  // together are accepted and measure the same).
  const bool cooperative = CG == 2 && p.stream_k != 0;
  if (cooperative) {
    attr[n_attr].id = cudaLaunchAttributeCooperative;
    attr[n_attr].val.cooperative = 1;
    ++n_attr;
  } else {
    // Programmatic dependent launch: the kernel may be scheduled while its predecessor in the
    // stream drains; it waits (griddepcontrol.wait) before its first global access.
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  if (CG == 2) {
    int pairs = grid / 2;
    if (max_clusters > 0 && pairs > max_clusters) pairs = max_clusters;
    if (pairs < 1) pairs = 1;
    grid = 2 * pairs;
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 2; attr[n_attr].val.clusterDim.y = 1; attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  cfg.attrs = attr; cfg.numAttrs = n_attr;
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(v2::threads_for(EW));
  cfg.dynamicSmemBytes = L::kDynamicBytes;
  cfg.stream = stream;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, ta, tb, tr, td, p);
  if (e != cudaSuccess && cooperative) {
    // a driver that refuses the combination: launch as the other kernels are (the bounded waits
    // of the kernel still turn a missing partner into a status code, never into a hang)
    cudaGetLastError();
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    e = cudaLaunchKernelEx(&cfg, kernel, ta, tb, tr, td, p);
  }
  if (e != cudaSuccess) { cudaGetLastError(); return FUSEML_E_LAUNCH; }
  return FUSEML_OK;
}

// Which execution form of the epilogue program a launch uses (epi::kProg*): the straight-line
// forms need the exact op sequence with the row vector staged in shared memory (reserved == 1)
// and a matrix operand that is not a staged row vector.
static int classify_program(const GemmParams& p) {
  if (p.uses_saved) return epi::kProgGenericSaved;
  auto is = [&](int i, int32_t opcode) { return p.ops[i].opcode == opcode; };
  auto staged_vec = [&](int i) { return is(i, FUSEML_OP_ADD_T) && p.ops[i].reserved == 1; };
  auto matrix_add = [&](int i) { return is(i, FUSEML_OP_ADD_T) && (p.ops[i].reserved == 0 || p.ops[i].reserved == 3); };
  if (p.n_ops == 2 && staged_vec(0) && is(1, FUSEML_OP_GELU_ERF)) return epi::kProgBiasGelu;
  if (p.n_ops == 2 && staged_vec(0) && matrix_add(1)) return epi::kProgBiasAdd;
  if (p.n_ops == 3 && staged_vec(0) && is(1, FUSEML_OP_GELU_ERF_MUL_SIGMOID) && matrix_add(2)) return epi::kProgBiasGeluSigAdd;
  return epi::kProgGeneric;
}

template <int BN, int STAGES, int CG, int EW = 8>
static int launch_bn(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tr, const CUtensorMap& td,
                     const GemmParams& p, int layout, int grid, cudaStream_t stream) {
  // layout: 0 = A and B K-major, 1 = B MN-major, 2 = A and B MN-major (see the kernel)
#define FUSEML_DISPATCH(PROG)                                                                             \
  case PROG:                                                                                              \
    return layout == 2 ? launch_instance<BN, STAGES, 2, PROG, CG, EW>(ta, tb, tr, td, p, grid, stream)    \
         : layout == 1 ? launch_instance<BN, STAGES, 1, PROG, CG, EW>(ta, tb, tr, td, p, grid, stream)    \
                       : launch_instance<BN, STAGES, 0, PROG, CG, EW>(ta, tb, tr, td, p, grid, stream)
  switch (classify_program(p)) {
    FUSEML_DISPATCH(epi::kProgGenericSaved);
    FUSEML_DISPATCH(epi::kProgBiasGelu);
    FUSEML_DISPATCH(epi::kProgBiasAdd);
    FUSEML_DISPATCH(epi::kProgBiasGeluSigAdd);
    default:
      FUSEML_DISPATCH(epi::kProgGeneric);
  }
#undef FUSEML_DISPATCH
}

// The pass that folds split-K (or small-MLP) partial tiles and runs the epilogue program.  Few
// tiles: eight columns per thread instead of sixteen, so that twice as many threads share the
// latency of reading the slices.
static int launch_finish(const GemmParams& pf, int64_t num_tiles, int bn, cudaStream_t stream) {
  const int64_t items16 = num_tiles * kTileM * (bn / 16);
  if (items16 < 148 * 256 * 2) {
    const int blocks = static_cast<int>((2 * items16 + 255) / 256);
    if (pf.uses_saved) splitk_finish_kernel<true, 8><<<blocks, 256, 0, stream>>>(pf);
    else splitk_finish_kernel<false, 8><<<blocks, 256, 0, stream>>>(pf);
  } else {
    const int blocks = static_cast<int>((items16 + 255) / 256);
    if (pf.uses_saved) splitk_finish_kernel<true, 16><<<blocks, 256, 0, stream>>>(pf);
    else splitk_finish_kernel<false, 16><<<blocks, 256, 0, stream>>>(pf);
  }
  return cudaGetLastError() == cudaSuccess ? FUSEML_OK : FUSEML_E_LAUNCH;
}

// Peephole over the epilogue program: the diamond gelu_erf(h) * sigmoid(h), written with the
// second value register as SAVE, GELU_ERF, SWAP, SIGMOID, MUL_SAVED (or with the two branches
// the other way round), becomes the single op FUSEML_OP_GELU_ERF_MUL_SIGMOID, which shares one
// reciprocal between the two functions.  Only when `saved` is not read again before the next
// SAVE: the fused op leaves it untouched.  Returns the new length.
static int fuse_diamonds(const fuseml_epi_op_t* in, int n, fuseml_epi_op_t* out) {
  int m = 0;
  for (int i = 0; i < n; ++i) {
    if (i + 4 < n && in[i].opcode == FUSEML_OP_SAVE && in[i + 2].opcode == FUSEML_OP_SWAP &&
        in[i + 4].opcode == FUSEML_OP_MUL_SAVED &&
        ((in[i + 1].opcode == FUSEML_OP_GELU_ERF && in[i + 3].opcode == FUSEML_OP_SIGMOID) ||
         (in[i + 1].opcode == FUSEML_OP_SIGMOID && in[i + 3].opcode == FUSEML_OP_GELU_ERF))) {
      bool dead = true;
      for (int j = i + 5; j < n; ++j) {
        const int32_t oc = in[j].opcode;
        if (oc == FUSEML_OP_SAVE) break;
        if (oc == FUSEML_OP_SWAP || oc == FUSEML_OP_ADD_SAVED || oc == FUSEML_OP_MUL_SAVED) { dead = false; break; }
      }
      if (dead) {
        out[m] = in[i];
        out[m].opcode = FUSEML_OP_GELU_ERF_MUL_SIGMOID;
        out[m].slot = 0;
        out[m].imm = 0.0f;
        ++m;
        i += 4;
        continue;
      }
    }
    out[m++] = in[i];
  }
  return m;
}

static int check_plan(const fuseml_plan_t* pl) {
  if (pl->tile_m != 128) return FUSEML_E_PLAN;
  if (pl->tile_n < 32 || pl->tile_n > 256 || pl->tile_n % 32 != 0) return FUSEML_E_PLAN;
  if (pl->grid <= 0 || pl->group_m <= 0) return FUSEML_E_PLAN;
  if (pl->cluster != 1 && pl->cluster != 2) return FUSEML_E_PLAN;
  if (pl->cluster == 2 && pl->tile_n <= 128) return FUSEML_E_PLAN;
  if (pl->split_k < 0 || pl->split_k > 64 || (pl->flags & ~(FUSEML_PLAN_B_EXPANSION_VALID | FUSEML_PLAN_STREAM_K | FUSEML_PLAN_GROUP_N)) != 0)
    return FUSEML_E_PLAN;
  if ((pl->flags & FUSEML_PLAN_STREAM_K) && (pl->cluster != 2 || pl->split_k > 1)) return FUSEML_E_PLAN;
  if (pl->split_k > 1 && pl->cluster != 1) return FUSEML_E_PLAN;
  return FUSEML_OK;
}

static int run_finalize(const fuseml_reduce_t& r, const WorkspaceLayout& w, char* ws, int64_t count,
                        cudaStream_t stream) {
  const float* psum = (r.kinds & (FUSEML_RED_SUM | FUSEML_RED_MEAN)) ? reinterpret_cast<float*>(ws + w.red_sum_off) : nullptr;
  const float* pmax = (r.kinds & FUSEML_RED_MAX) ? reinterpret_cast<float*>(ws + w.red_max_off) : nullptr;
  float* o_sum = (r.kinds & FUSEML_RED_SUM) ? r.out_sum : nullptr;
  float* o_max = (r.kinds & FUSEML_RED_MAX) ? r.out_max : nullptr;
  float* o_mean = (r.kinds & FUSEML_RED_MEAN) ? r.out_mean : nullptr;
  const int threads = 256;
  const int blocks = w.len == 1 ? 1 : static_cast<int>(std::min<int64_t>((w.len + threads - 1) / threads, 1184));
  reduce_finalize_kernel<<<blocks, threads, 0, stream>>>(psum, pmax, w.partials, w.len, 1.0 / static_cast<double>(count),
                                                         o_sum, o_max, o_mean);
  return cudaGetLastError() == cudaSuccess ? FUSEML_OK : FUSEML_E_LAUNCH;
}

}  // namespace fuseml

using namespace fuseml;

extern "C" {

int fuseml_sm100_abi_version(void) { return FUSEML_SM100_ABI_VERSION; }

const char* fuseml_sm100_strerror(int code) {
  switch (code) {
    case FUSEML_OK: return "ok";
    case FUSEML_E_NULL: return "a required pointer is null";
    case FUSEML_E_SHAPE: return "M, N and K must be positive and below 2^31";
    case FUSEML_E_DTYPE: return "unsupported dtype";
    case FUSEML_E_LAYOUT: return "layout not supported: bases must be 16-byte aligned, one unit stride per matrix, leading strides multiples of 16 bytes";
    case FUSEML_E_EPILOGUE: return "bad epilogue program (opcode, operand slot or length)";
    case FUSEML_E_REDUCTION: return "bad reduction request";
    case FUSEML_E_WORKSPACE: return "workspace missing or too small (see fuseml_sm100_workspace_bytes)";
    case FUSEML_E_PLAN: return "plan fields out of range";
    case FUSEML_E_DEVICE: return "no sm_100 CUDA device or driver entry point unavailable";
    case FUSEML_E_LAUNCH: return "CUDA reported an error at launch";
    case FUSEML_E_TIMEOUT: return "a bounded device-side wait ran out";
    case FUSEML_E_LIMIT: return "size beyond a documented fixed maximum";
    default: return "unknown fuseml status code";
  }
}

int fuseml_sm100_query(fuseml_device_props_t* props) {
  if (props == nullptr) return FUSEML_E_NULL;
  default_props(props);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return FUSEML_E_DEVICE; }
  cudaDeviceProp dp;
  if (cudaGetDeviceProperties(&dp, dev) != cudaSuccess) { cudaGetLastError(); return FUSEML_E_DEVICE; }
  props->sm_count = dp.multiProcessorCount;
  props->cc_major = dp.major;
  props->cc_minor = dp.minor;
  props->smem_per_block_optin = static_cast<int32_t>(dp.sharedMemPerBlockOptin);
  props->l2_bytes = dp.l2CacheSize;
  return dp.major == 10 ? FUSEML_OK : FUSEML_E_DEVICE;
}

int fuseml_sm100_plan(const fuseml_gemm_desc_t* desc, const fuseml_device_props_t* props, fuseml_plan_t* plan) {
  return make_plan(desc, props, plan);
}

int fuseml_sm100_validate(const fuseml_gemm_desc_t* desc) { return validate_desc(desc); }

int64_t fuseml_sm100_workspace_bytes(const fuseml_gemm_desc_t* desc, const fuseml_plan_t* plan) {
  if (desc == nullptr) return -1;
  fuseml_plan_t local;
  if (plan == nullptr) {
    if (make_plan(desc, nullptr, &local) != FUSEML_OK) return -1;
  } else {
    // a caller's plan is checked before any arithmetic divides by its tile shape
    if (validate_desc(desc) != FUSEML_OK || check_plan(plan) != FUSEML_OK) return -1;
    local = *plan;
  }
  if (local.split_k < 1) local.split_k = 1;
  WorkspaceLayout w;
  workspace_layout(desc, &local, &w);
  return w.total;
}

int fuseml_sm100_gemm_epilogue(const fuseml_gemm_desc_t* desc, const fuseml_plan_t* plan_in, void* cuda_stream) {
  int rc = validate_desc(desc);
  if (rc != FUSEML_OK) return rc;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);

  fuseml_plan_t plan;
  if (plan_in != nullptr) {
    plan = *plan_in;
  } else {
    fuseml_device_props_t props;
    if (fuseml_sm100_query(&props) != FUSEML_OK) return FUSEML_E_DEVICE;
    rc = make_plan(desc, &props, &plan);
    if (rc != FUSEML_OK) return rc;
  }
  rc = check_plan(&plan);
  if (rc != FUSEML_OK) return rc;
  if (plan.split_k < 1) plan.split_k = 1;     // a zero-initialised plan means "no split"
  // split-K has no fused reductions and needs an output to write
  if (plan.split_k > 1 && (desc->reduce.kinds != 0 || desc->d == nullptr)) return FUSEML_E_PLAN;

  WorkspaceLayout w;
  workspace_layout(desc, &plan, &w);
  char* ws = reinterpret_cast<char*>(desc->reduce.workspace);
  if (w.total > 0) {
    if (ws == nullptr || desc->reduce.workspace_bytes < w.total) return FUSEML_E_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(ws) & 15u) != 0) return FUSEML_E_WORKSPACE;
  }

  const bool f32 = desc->ab_dtype == FUSEML_F32;
  const int fmt = f32 ? 2 : (desc->ab_dtype == FUSEML_BF16 ? 1 : 0);
  const int bl = b_layout(desc);
  const void* a_ptr = desc->a;
  const void* b_ptr = desc->b;
  bool a_mn = a_layout(desc) == 1;
  int64_t K = desc->K, lda = a_mn ? desc->a_stride_k : desc->lda, ldb = (bl == 0) ? desc->b_stride_n : desc->b_stride_k;
  bool b_mn = (bl == 1);
  if (f32) {
    // expand both operands to [rows, 3K] K-major copies in the workspace
    const int64_t ld = split_ld(desc->K);
    float* a2 = reinterpret_cast<float*>(ws + w.split_a_off);
    float* b2 = reinterpret_cast<float*>(ws + w.split_b_off);
    const int threads = 256;
    const int64_t ta = desc->M * desc->K, tb = desc->N * desc->K;
    SplitJob ja = {reinterpret_cast<const float*>(desc->a), desc->M, desc->K, desc->lda, a_mn ? desc->a_stride_k : 1, 0, a2, ld,
                   static_cast<int32_t>(std::min<int64_t>((ta + threads - 1) / threads, 148 * 8))};
    SplitJob jb = {reinterpret_cast<const float*>(desc->b), desc->N, desc->K, desc->b_stride_n, desc->b_stride_k, 1, b2, ld,
                   static_cast<int32_t>(std::min<int64_t>((tb + threads - 1) / threads, 148 * 8))};
    if (plan.flags & FUSEML_PLAN_B_EXPANSION_VALID) jb.blocks = 0;
    // one launch for both operands
    SplitJob none = {};
    split_tf32_kernel<<<ja.blocks + jb.blocks, threads, 0, stream>>>(ja, jb, none);
    if (cudaGetLastError() != cudaSuccess) return FUSEML_E_LAUNCH;
    a_ptr = a2; b_ptr = b2; K = 3 * desc->K; lda = ld; ldb = ld; b_mn = false; a_mn = false;
  }
  const int layout = a_mn ? 2 : (b_mn ? 1 : 0);

  const int BN = plan.tile_n;          // run-time tile width; kernels are built for 128 and 256
  const int BK = f32 ? 32 : 64;
  CUtensorMap ta, tb;
  if (!a_mn) rc = encode_2d(&ta, desc->ab_dtype, a_ptr, desc->M, K, lda, BK, kTileM);
  else rc = encode_2d(&ta, desc->ab_dtype, a_ptr, K, desc->M, lda, 64, BK);     // stored [K, M]: boxes of 64 k x 64 m
  if (rc != FUSEML_OK) return rc;
  // K-major B: one box per CTA covers that CTA's share of the tile's columns (all of them for a
  // single CTA, half for a CTA pair)
  if (!b_mn) rc = encode_2d(&tb, desc->ab_dtype, b_ptr, desc->N, K, ldb, BK, BN / plan.cluster);
  else rc = encode_2d(&tb, desc->ab_dtype, b_ptr, K, desc->N, ldb, 64, BK);
  if (rc != FUSEML_OK) return rc;

  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.M = static_cast<int32_t>(desc->M);
  p.N = static_cast<int32_t>(desc->N);
  p.K = static_cast<int32_t>(K);
  const int CGr = plan.cluster;
  p.fmt = fmt;
  p.tiles_m = static_cast<int32_t>((desc->M + kTileM * CGr - 1) / (kTileM * CGr));
  p.tiles_n = static_cast<int32_t>((desc->N + BN - 1) / BN);
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.bn = BN;
  p.group_m = (plan.flags & FUSEML_PLAN_GROUP_N) ? -std::min(plan.group_m, p.tiles_n) : std::min(plan.group_m, p.tiles_m);
  p.num_kb = static_cast<int32_t>((K + BK - 1) / BK);
  p.d = desc->d;
  p.ldd = desc->ldd;
  p.out_dtype = desc->out_dtype;
  p.n_ops = fuse_diamonds(desc->ops, desc->n_ops, p.ops);
  for (int i = 0; i < p.n_ops; ++i) {
    p.ops[i].reserved = 0;
    const int32_t oc = p.ops[i].opcode;
    if (oc == FUSEML_OP_SAVE || oc == FUSEML_OP_SWAP || oc == FUSEML_OP_ADD_SAVED || oc == FUSEML_OP_MUL_SAVED)
      p.uses_saved = 1;
  }
  for (int i = 0; i < desc->n_operands; ++i) {
    p.operands[i].ptr = desc->operands[i].ptr;
    p.operands[i].stride_m = desc->operands[i].stride_m;
    p.operands[i].stride_n = desc->operands[i].stride_n;
    p.operands[i].dtype = desc->operands[i].dtype;
  }
  // operands fetched ahead of use (see GemmParams): row vectors staged in shared memory, the
  // first 16-byte-loadable 16-bit matrix operand requested at the top of each chunk
  p.vec_slot[0] = p.vec_slot[1] = -1;
  p.mat_slot = -1;
  {
    int n_vec = 0;
    for (int i = 0; i < p.n_ops; ++i) {
      const int32_t oc = p.ops[i].opcode;
      if (oc != FUSEML_OP_ADD_T && oc != FUSEML_OP_MUL_T) continue;
      const int32_t slot = p.ops[i].slot;
      const fuseml_operand_t& o = desc->operands[slot];
      if (o.stride_m == 0 && o.stride_n == 1) {
        int idx = -1;
        for (int j = 0; j < n_vec; ++j) if (p.vec_slot[j] == slot) idx = j;
        if (idx < 0 && n_vec < 2) { idx = n_vec; p.vec_slot[n_vec++] = slot; }
        if (idx >= 0) p.ops[i].reserved = idx + 1;
      } else if (o.stride_n == 1 && (o.dtype == FUSEML_BF16 || o.dtype == FUSEML_F16) &&
                 (reinterpret_cast<uintptr_t>(o.ptr) & 15u) == 0 && (o.stride_m * 2) % 16 == 0 &&
                 (p.mat_slot < 0 || p.mat_slot == slot)) {
        p.mat_slot = slot;
        p.ops[i].reserved = 3;
      }
    }
  }
  // an operand whose every element is read by at most two tile units is a pure stream
  p.a_stream = p.b_stream = 0;
  if (p.tiles_m <= 2 && p.tiles_n > 2) { p.b_stream = 1; p.a_stream = 2; }
  else if (p.tiles_n <= 2 && p.tiles_m > 2) { p.a_stream = 1; p.b_stream = 2; }
  p.red_kinds = desc->reduce.kinds;
  p.red_axis = desc->reduce.axis;
  if (desc->reduce.kinds != 0) {
    if (desc->reduce.kinds & (FUSEML_RED_SUM | FUSEML_RED_MEAN)) p.red_sum = reinterpret_cast<float*>(ws + w.red_sum_off);
    if (desc->reduce.kinds & FUSEML_RED_MAX) p.red_max = reinterpret_cast<float*>(ws + w.red_max_off);
  }
  void* status_ptr = nullptr;
  if (cudaGetSymbolAddress(&status_ptr, g_status_word) != cudaSuccess) { cudaGetLastError(); return FUSEML_E_DEVICE; }
  p.status = reinterpret_cast<int32_t*>(status_ptr);
  p.wait_limit_us = g_diag_wait_limit_us.load(std::memory_order_relaxed);
  p.drop_last_load = g_diag_drop_last_load.load(std::memory_order_relaxed);

  if (plan.split_k > 1) {
    // Split-K: every CTA runs one K slice of one tile and stores its raw fp32 accumulator; the
    // epilogue program runs in splitk_finish_kernel on the folded slices.
    const int32_t per = (p.num_kb + plan.split_k - 1) / plan.split_k;
    const int32_t slices = (p.num_kb + per - 1) / per;          // none of them empty
    GemmParams pg = p;
    pg.split_k = slices;
    pg.kb_per_split = per;
    pg.split_ws = reinterpret_cast<float*>(ws + w.splitk_off);
    pg.n_ops = 0;
    pg.uses_saved = 0;
    pg.vec_slot[0] = pg.vec_slot[1] = -1;
    pg.mat_slot = -1;
    CUtensorMap none;
    std::memset(&none, 0, sizeof(none));
    const int items = p.num_tiles * slices;
    if (slices > 1) {
      if (BN > 128) rc = launch_bn<256, 4, 1>(ta, tb, none, none, pg, layout, items, stream);
      else rc = launch_bn<128, 6, 1>(ta, tb, none, none, pg, layout, items, stream);
      if (rc != FUSEML_OK) return rc;
      GemmParams pf = p;
      pf.split_k = slices;
      pf.kb_per_split = per;
      pf.split_ws = pg.split_ws;
      for (int i = 0; i < pf.n_ops; ++i) pf.ops[i].reserved = 0;   // operands come straight from global memory
      // an ordinary launch: as a programmatic dependent (scheduled early, waiting on the device)
      // it measured 20-35 % slower at high slice counts
      return launch_finish(pf, p.num_tiles, BN, stream);
    }
  }

  // (programs with a second value register run whole tiles only: see kStreamK in the kernel)
  const bool stream_k = (plan.flags & FUSEML_PLAN_STREAM_K) != 0 && !p.uses_saved;
  int grid = stream_k ? plan.grid : std::min(plan.grid, p.num_tiles * CGr);
  if (stream_k) {
    p.stream_k = 1;
    p.sk_ws = reinterpret_cast<float*>(ws + w.sk_ws_off);
    p.sk_flags = reinterpret_cast<uint32_t*>(ws + w.sk_flags_off);
    if (cudaMemsetAsync(p.sk_flags, 0, static_cast<size_t>(w.sk_flags_bytes), stream) != cudaSuccess) { cudaGetLastError(); return FUSEML_E_LAUNCH; }
  }
  if (desc->reduce.kinds != 0 && desc->reduce.axis == FUSEML_AXIS_ALL) {
    // AXIS_ALL partials: one per launched CTA.  Slots of CTAs that end up not launched (the
    // device holds fewer CTA pairs than asked for) are filled with neutral values first.
    grid = std::min<int>(grid, static_cast<int>(w.partials));
    fill_neutral_kernel<<<1, 256, 0, stream>>>(p.red_sum, p.red_max, static_cast<int>(w.partials));
  }
  // A launch in which no CTA gets a second tile has nothing to overlap its epilogue with: run it
  // with sixteen epilogue warps on 16-column chunks (twice the warps in flight for the operand
  // loads, the special-function unit and the stores).  Reductions keep the 8-warp instance
  // (their partial layout is sized for two warps per row).
  const bool lone_tile = p.num_tiles * CGr <= grid && p.red_kinds == 0 && fmt != 2 && !stream_k;
  CUtensorMap tr, td;
  std::memset(&tr, 0, sizeof(tr));
  std::memset(&td, 0, sizeof(td));
  // tile I/O needs whole 64-column boxes; the sixteen-warp instances exist for the full-width
  // pair kernel and for both single-CTA kernels
  const bool staged = lone_tile && BN % 64 == 0 && (CGr == 1 || BN == 256);
  if (staged) {
    // Tile I/O through shared memory: the matrix operand (residual) and the output tile move
    // as 128 x 64 boxes by TMA instead of row-per-thread accesses.  16-bit types, 16-byte
    // aligned base and row pitch (what a tensor map needs); anything else keeps the direct path.
    if (p.mat_slot >= 0) {
      const EpiOperand& mo = p.operands[p.mat_slot];
      if (encode_2d(&tr, mo.dtype, mo.ptr, desc->M, desc->N, mo.stride_m, 64, kTileM) == FUSEML_OK) p.io_flags |= 1;
    }
    if (p.d != nullptr && (p.out_dtype == FUSEML_BF16 || p.out_dtype == FUSEML_F16) &&
        (reinterpret_cast<uintptr_t>(p.d) & 15u) == 0 && (p.ldd * 2) % 16 == 0 &&
        encode_2d(&td, p.out_dtype, p.d, desc->M, desc->N, p.ldd, 64, kTileM) == FUSEML_OK) {
      p.io_flags |= 2;
    }
    if (CGr == 2) rc = launch_bn<256, 6, 2, 16>(ta, tb, tr, td, p, layout, grid, stream);
    else if (BN > 128) rc = launch_bn<256, 4, 1, 16>(ta, tb, tr, td, p, layout, grid, stream);
    else rc = launch_bn<128, 6, 1, 16>(ta, tb, tr, td, p, layout, grid, stream);
  } else if (CGr == 2) rc = launch_bn<256, 6, 2>(ta, tb, tr, td, p, layout, grid, stream);
  else if (BN > 128) rc = launch_bn<256, 4, 1>(ta, tb, tr, td, p, layout, grid, stream);
  else rc = launch_bn<128, 6, 1>(ta, tb, tr, td, p, layout, grid, stream);
  if (rc != FUSEML_OK) return rc;

  if (desc->reduce.kinds != 0) {
    const int64_t count = desc->reduce.axis == FUSEML_AXIS_N ? desc->N
                        : desc->reduce.axis == FUSEML_AXIS_M ? desc->M : desc->M * desc->N;
    rc = run_finalize(desc->reduce, w, ws, count, stream);
  }
  return rc;
}

// ---- small-M MLP block in one kernel --------------------------------------------------------
namespace fuseml {

struct MlpLayout {
  int32_t bi, groups, n_dchunks, slices;
  int64_t x_off, w1_off, w2_off, part_off, total;   // workspace (the first three: fp32 expansions)
  int64_t ld1, ld2;                                 // leading dimensions of the expansions
};

static bool mlp_uses(const fuseml_epi_op_t* ops, int n, std::initializer_list<int32_t> codes) {
  for (int i = 0; i < n; ++i)
    for (int32_t c : codes)
      if (ops[i].opcode == c) return true;
  return false;
}

// FUSEML_OK and the layout, or the reason the block cannot run as one kernel.
static int mlp_layout(const fuseml_mlp_desc_t* d, MlpLayout* L) {
  if (d == nullptr) return FUSEML_E_NULL;
  if (d->x == nullptr || d->w1 == nullptr || d->w2 == nullptr || d->y == nullptr) return FUSEML_E_NULL;
  if (d->M <= 0 || d->D_in <= 0 || d->I <= 0 || d->D_out <= 0) return FUSEML_E_SHAPE;
  if (d->M > 128 || d->D_in > (1 << 24) || d->I > (1 << 24) || d->D_out > (1 << 24)) return FUSEML_E_SHAPE;
  const int eb = dtype_bytes(d->ab_dtype);
  if (eb == 0 || dtype_bytes(d->out_dtype) == 0) return FUSEML_E_DTYPE;
  const bool f32 = d->ab_dtype == FUSEML_F32;
  if (d->ldx < d->D_in || d->ldw1 < d->D_in || d->ldw2 < d->I || d->ldy < d->D_out) return FUSEML_E_LAYOUT;
  if (!f32) {
    for (const void* p : {d->x, d->w1, d->w2})
      if (reinterpret_cast<uintptr_t>(p) & 15u) return FUSEML_E_LAYOUT;
    if ((d->ldx * eb) % 16 || (d->ldw1 * eb) % 16 || (d->ldw2 * eb) % 16) return FUSEML_E_LAYOUT;
  } else if (d->I % 4 != 0) {
    return FUSEML_E_LAYOUT;             // the three copies of an expanded row must start on 16-byte boundaries
  }
  if (d->n_ops1 < 0 || d->n_ops1 > FUSEML_MAX_EPI_OPS || d->n_ops2 < 0 || d->n_ops2 > FUSEML_MAX_EPI_OPS ||
      d->n_operands < 0 || d->n_operands > FUSEML_MAX_OPERANDS)
    return FUSEML_E_EPILOGUE;
  for (int pass = 0; pass < 2; ++pass) {
    const fuseml_epi_op_t* ops = pass ? d->ops2 : d->ops1;
    const int n = pass ? d->n_ops2 : d->n_ops1;
    for (int i = 0; i < n; ++i) {
      const int32_t oc = ops[i].opcode;
      if (oc < 0 || oc >= FUSEML_OP__COUNT) return FUSEML_E_EPILOGUE;
      const bool uses = oc == FUSEML_OP_ADD_T || oc == FUSEML_OP_MUL_T || oc == FUSEML_OP_SUB_T || oc == FUSEML_OP_RSUB_T ||
                        oc == FUSEML_OP_STORE_AUX || oc == FUSEML_OP_GELU_ERF_BWD_T;
      if (uses) {
        if (ops[i].slot < 0 || ops[i].slot >= d->n_operands) return FUSEML_E_EPILOGUE;
        const fuseml_operand_t& o = d->operands[ops[i].slot];
        if (o.ptr == nullptr) return FUSEML_E_NULL;
        if (dtype_bytes(o.dtype) == 0) return FUSEML_E_DTYPE;
        if (o.stride_m < 0 || o.stride_n < 0) return FUSEML_E_LAYOUT;
      }
    }
  }
  // the first program runs in the interpreter without the second register and without escape stores
  fuseml_epi_op_t tmp[FUSEML_MAX_EPI_OPS];
  const int n1 = fuse_diamonds(d->ops1, d->n_ops1, tmp);
  if (mlp_uses(tmp, n1, {FUSEML_OP_SAVE, FUSEML_OP_SWAP, FUSEML_OP_ADD_SAVED, FUSEML_OP_MUL_SAVED, FUSEML_OP_STORE_AUX}))
    return FUSEML_E_EPILOGUE;
  // slice width: the widest of the candidates that divides I
  const int cands[2] = {f32 ? 64 : 128, f32 ? 32 : 64};
  int bi = 0;
  for (int c : cands)
    if (bi == 0 && d->I % c == 0) bi = c;
  if (bi == 0) return FUSEML_E_SHAPE;
  L->bi = bi;
  L->slices = static_cast<int32_t>(d->I / bi);
  L->n_dchunks = static_cast<int32_t>((d->D_out + 255) / 256);
  // every 256-column chunk of the output recomputes h for its slices: beyond two chunks the
  // repeated first GEMM costs more than a trip of h through L2 (measured: 128 x 4096 x 16384 x 4096
  // takes 800 us this way against 58 us as two launches)
  if (L->n_dchunks > 2) return FUSEML_E_SHAPE;
  // CTAs per output chunk: one per slice if they fit the machine; the partial tiles (128 KB per CTA) stay within 8 MiB
  const int per_chunk = std::max(1, std::min(148, 64) / L->n_dchunks);
  L->groups = std::max(1, std::min(L->slices, per_chunk));
  if (static_cast<int64_t>(L->groups) * L->n_dchunks > 148) return FUSEML_E_SHAPE;
  int64_t off = 0;
  auto take = [&](int64_t bytes) { const int64_t at = off; off += (bytes + 255) / 256 * 256; return at; };
  L->ld1 = split_ld(d->D_in);
  L->ld2 = split_ld(d->I);
  L->x_off = L->w1_off = L->w2_off = 0;
  if (f32) {
    L->x_off = take(d->M * L->ld1 * 4);
    L->w1_off = take(d->I * L->ld1 * 4);
    L->w2_off = take(d->D_out * L->ld2 * 4);
  }
  L->part_off = take(static_cast<int64_t>(L->groups) * L->n_dchunks * 128 * 256 * 4);
  L->total = off;
  return FUSEML_OK;
}

}  // namespace fuseml

int64_t fuseml_sm100_mlp_small_workspace_bytes(const fuseml_mlp_desc_t* desc) {
  MlpLayout L;
  return mlp_layout(desc, &L) == FUSEML_OK ? L.total : -1;
}

int fuseml_sm100_mlp_small(const fuseml_mlp_desc_t* desc, void* cuda_stream) {
  MlpLayout L;
  int rc = mlp_layout(desc, &L);
  if (rc != FUSEML_OK) return rc;
  char* ws = reinterpret_cast<char*>(desc->workspace);
  if (ws == nullptr || desc->workspace_bytes < L.total || (reinterpret_cast<uintptr_t>(ws) & 15u)) return FUSEML_E_WORKSPACE;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
  const bool f32 = desc->ab_dtype == FUSEML_F32;
  const int fmt = f32 ? 2 : (desc->ab_dtype == FUSEML_BF16 ? 1 : 0);
  const int BK = f32 ? 32 : 64;

  const void* x = desc->x; const void* w1 = desc->w1; const void* w2 = desc->w2;
  int64_t K1 = desc->D_in, K2 = desc->I, ldx = desc->ldx, ldw1 = desc->ldw1, ldw2 = desc->ldw2;
  if (f32) {
    float* xe = reinterpret_cast<float*>(ws + L.x_off);
    float* w1e = reinterpret_cast<float*>(ws + L.w1_off);
    float* w2e = reinterpret_cast<float*>(ws + L.w2_off);
    const int threads = 256;
    auto blocks = [&](int64_t n) { return static_cast<int32_t>(std::min<int64_t>((n + threads - 1) / threads, 148 * 8)); };
    SplitJob jx = {reinterpret_cast<const float*>(desc->x), desc->M, desc->D_in, desc->ldx, 1, 0, xe, L.ld1, blocks(desc->M * desc->D_in)};
    SplitJob j1 = {reinterpret_cast<const float*>(desc->w1), desc->I, desc->D_in, desc->ldw1, 1, 1, w1e, L.ld1, blocks(desc->I * desc->D_in)};
    SplitJob j2 = {reinterpret_cast<const float*>(desc->w2), desc->D_out, desc->I, desc->ldw2, 1, 1, w2e, L.ld2, blocks(desc->D_out * desc->I)};
    if (desc->flags & FUSEML_MLP_WEIGHTS_EXPANDED) j1.blocks = j2.blocks = 0;
    split_tf32_kernel<<<jx.blocks + j1.blocks + j2.blocks, threads, 0, stream>>>(jx, j1, j2);
    if (cudaGetLastError() != cudaSuccess) return FUSEML_E_LAUNCH;
    x = xe; w1 = w1e; w2 = w2e; K1 = 3 * desc->D_in; K2 = 3 * desc->I; ldx = ldw1 = L.ld1; ldw2 = L.ld2;
  }
  CUtensorMap tx, t1, t2;
  if ((rc = encode_2d(&tx, desc->ab_dtype, x, desc->M, K1, ldx, BK, 128)) != FUSEML_OK) return rc;
  if ((rc = encode_2d(&t1, desc->ab_dtype, w1, desc->I, K1, ldw1, BK, L.bi)) != FUSEML_OK) return rc;
  if ((rc = encode_2d(&t2, desc->ab_dtype, w2, desc->D_out, K2, ldw2, BK, 128)) != FUSEML_OK) return rc;

  void* status_ptr = nullptr;
  if (cudaGetSymbolAddress(&status_ptr, g_status_word) != cudaSuccess) { cudaGetLastError(); return FUSEML_E_DEVICE; }

  mlp::MlpParams q;
  std::memset(&q, 0, sizeof(q));
  q.M = static_cast<int32_t>(desc->M);
  q.I = static_cast<int32_t>(desc->I);
  q.D_out = static_cast<int32_t>(desc->D_out);
  q.fmt = fmt;
  q.bi = L.bi;
  q.num_slices = L.slices;
  q.groups = L.groups;
  q.n_dchunks = L.n_dchunks;
  q.kb1 = static_cast<int32_t>((K1 + BK - 1) / BK);
  q.out16 = desc->ab_dtype == FUSEML_F16 ? 1 : 0;
  q.split_ws = reinterpret_cast<float*>(ws + L.part_off);
  q.status = reinterpret_cast<int32_t*>(status_ptr);
  q.wait_limit_us = g_diag_wait_limit_us.load(std::memory_order_relaxed);

  // program 1 runs on h[M, I]; program 2 (in the finish pass) on y[M, D_out]
  GemmParams p1, p2;
  std::memset(&p1, 0, sizeof(p1));
  std::memset(&p2, 0, sizeof(p2));
  for (GemmParams* p : {&p1, &p2}) {
    for (int i = 0; i < desc->n_operands; ++i) {
      p->operands[i].ptr = desc->operands[i].ptr;
      p->operands[i].stride_m = desc->operands[i].stride_m;
      p->operands[i].stride_n = desc->operands[i].stride_n;
      p->operands[i].dtype = desc->operands[i].dtype;
    }
    p->M = q.M;
    p->vec_slot[0] = p->vec_slot[1] = -1;
    p->mat_slot = -1;
    p->status = q.status;
  }
  p1.N = q.I;
  p1.n_ops = fuse_diamonds(desc->ops1, desc->n_ops1, p1.ops);
  p2.N = q.D_out;
  p2.n_ops = fuse_diamonds(desc->ops2, desc->n_ops2, p2.ops);
  for (int i = 0; i < p1.n_ops; ++i) p1.ops[i].reserved = 0;
  for (int i = 0; i < p2.n_ops; ++i) {
    p2.ops[i].reserved = 0;
    const int32_t oc = p2.ops[i].opcode;
    if (oc == FUSEML_OP_SAVE || oc == FUSEML_OP_SWAP || oc == FUSEML_OP_ADD_SAVED || oc == FUSEML_OP_MUL_SAVED) p2.uses_saved = 1;
  }
  p2.tiles_m = 1;
  p2.tiles_n = p2.num_tiles = L.n_dchunks;
  p2.group_m = 1;
  p2.bn = 256;
  p2.d = desc->y;
  p2.ldd = desc->ldy;
  p2.out_dtype = desc->out_dtype;
  p2.split_k = L.groups;
  p2.split_ws = q.split_ws;

  const int smem_bytes = f32 ? mlp::Layout<true>::kDynamicBytes : mlp::Layout<false>::kDynamicBytes;
  {
    static std::mutex mutex;
    static bool configured[kMaxDevices] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return FUSEML_E_DEVICE; }
    std::lock_guard<std::mutex> lock(mutex);
    if (!configured[dev]) {
      if (cudaFuncSetAttribute(mlp::mlp_small_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               mlp::Layout<true>::kDynamicBytes) != cudaSuccess ||
          cudaFuncSetAttribute(mlp::mlp_small_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               mlp::Layout<false>::kDynamicBytes) != cudaSuccess) {
        cudaGetLastError();
        return FUSEML_E_LAUNCH;
      }
      configured[dev] = true;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  cfg.gridDim = dim3(L.groups * L.n_dchunks);
  cfg.blockDim = dim3(mlp::kThreads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  const cudaError_t le = f32 ? cudaLaunchKernelEx(&cfg, mlp::mlp_small_kernel<true>, tx, t1, t2, q, p1)
                             : cudaLaunchKernelEx(&cfg, mlp::mlp_small_kernel<false>, tx, t1, t2, q, p1);
  if (le != cudaSuccess) { cudaGetLastError(); return FUSEML_E_LAUNCH; }

  return launch_finish(p2, L.n_dchunks, 256, stream);
}

int fuseml_sm100_reduce_tail(const void* x, int32_t dtype, int64_t M, int64_t N, int64_t ldx,
                             const fuseml_reduce_t* r, void* cuda_stream) {
  if (x == nullptr || r == nullptr) return FUSEML_E_NULL;
  if (M <= 0 || N <= 0 || ldx < N) return FUSEML_E_SHAPE;
  if (dtype_bytes(dtype) == 0) return FUSEML_E_DTYPE;
  if (r->kinds == 0 || (r->kinds & ~7)) return FUSEML_E_REDUCTION;
  if ((r->kinds & FUSEML_RED_SUM) && !r->out_sum) return FUSEML_E_NULL;
  if ((r->kinds & FUSEML_RED_MAX) && !r->out_max) return FUSEML_E_NULL;
  if ((r->kinds & FUSEML_RED_MEAN) && !r->out_mean) return FUSEML_E_NULL;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
  const bool want_sum = (r->kinds & (FUSEML_RED_SUM | FUSEML_RED_MEAN)) != 0;
  const bool want_max = (r->kinds & FUSEML_RED_MAX) != 0;
  if (r->axis == FUSEML_AXIS_N) {
    const int grid = static_cast<int>(std::min<int64_t>(M, 148 * 8));
    reduce_rows_kernel<<<grid, 256, 0, stream>>>(x, dtype, M, N, ldx, 0, 1.0 / static_cast<double>(N),
                                                 (r->kinds & FUSEML_RED_SUM) ? r->out_sum : nullptr,
                                                 want_max ? r->out_max : nullptr,
                                                 (r->kinds & FUSEML_RED_MEAN) ? r->out_mean : nullptr);
    return cudaGetLastError() == cudaSuccess ? FUSEML_OK : FUSEML_E_LAUNCH;
  }
  // partials through the workspace
  WorkspaceLayout w;
  std::memset(&w, 0, sizeof(w));
  int64_t rows_per_slice = 0;
  if (r->axis == FUSEML_AXIS_ALL) { w.partials = std::min<int64_t>(M, 148 * 8); w.len = 1; }
  else if (r->axis == FUSEML_AXIS_M) {
    const int64_t slices = std::max<int64_t>(1, std::min<int64_t>((M + 63) / 64, 64));
    rows_per_slice = (M + slices - 1) / slices;
    w.partials = (M + rows_per_slice - 1) / rows_per_slice; w.len = N;
  } else return FUSEML_E_REDUCTION;
  int64_t off = 0;
  const int64_t each = ((w.partials * w.len * 4 + 255) / 256) * 256;
  if (want_sum) { w.red_sum_off = off; off += each; }
  if (want_max) { w.red_max_off = off; off += each; }
  char* ws = reinterpret_cast<char*>(r->workspace);
  if (ws == nullptr || r->workspace_bytes < off) return FUSEML_E_WORKSPACE;
  float* psum = want_sum ? reinterpret_cast<float*>(ws + w.red_sum_off) : nullptr;
  float* pmax = want_max ? reinterpret_cast<float*>(ws + w.red_max_off) : nullptr;
  if (r->axis == FUSEML_AXIS_ALL) {
    reduce_rows_kernel<<<static_cast<int>(w.partials), 256, 0, stream>>>(x, dtype, M, N, ldx, 1, 0.0, psum, pmax, nullptr);
  } else {
    dim3 grid(static_cast<unsigned>((N + 255) / 256), static_cast<unsigned>(w.partials));
    reduce_cols_kernel<<<grid, 256, 0, stream>>>(x, dtype, M, N, ldx, rows_per_slice, psum, pmax);
  }
  if (cudaGetLastError() != cudaSuccess) return FUSEML_E_LAUNCH;
  const int64_t count = r->axis == FUSEML_AXIS_M ? M : M * N;
  return run_finalize(*r, w, ws, count, stream);
}

// ---------------------------------------------------------------------------------
// Entry point for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the moment they need a fused
// GEMM with a reduction tail: code running inside another framework's memory pool
// with the allocator locked, a plugin that was handed a fixed memory budget at load
// time, or a latency-critical serving loop where an allocation (and the implicit
// synchronisation it can cause) is not acceptable.  For them the reduction partials
// live in the fixed array below instead of a caller-provided workspace.
//
// Cost and limits: every GPU that loads this library holds kNoAllocScratchBytes
// (8 MiB) of device memory until the process exits, whether or not this entry point
// is ever called.  A launch whose scratch need is larger is rejected with
// FUSEML_E_LIMIT.  The array is shared by every call: it keeps whatever the last
// call left there (the kernels overwrite every slot they later read, so nothing has
// to be cleared), and two calls whose kernels overlap on the GPU (different streams,
// or different host threads) race on it - serialise them on one stream.
// ---------------------------------------------------------------------------------
namespace fuseml {
constexpr int64_t kNoAllocScratchBytes = 8ll << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

static void* g_noalloc_ptr[kMaxDevices] = {nullptr};
static std::mutex g_noalloc_mutex;

// Device address of the scratch array on the current device.  `g_noalloc_scratch` in
// host code is only a handle for the symbol, not an address a kernel can use; the real
// address differs per device and is looked up once per device, with that device
// current, and cached.
static int noalloc_scratch_address(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return FUSEML_E_DEVICE; }
  if (dev < 0 || dev >= kMaxDevices) return FUSEML_E_DEVICE;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      return FUSEML_E_DEVICE;
    }
    g_noalloc_ptr[dev] = ptr;
  }
  *out = g_noalloc_ptr[dev];
  return FUSEML_OK;
}
}  // namespace fuseml

int64_t fuseml_sm100_noalloc_scratch_bytes(void) { return kNoAllocScratchBytes; }

// whether the program, after the diamond rewrite, still keeps a second value register
static bool program_uses_saved(const fuseml_gemm_desc_t* desc) {
  fuseml_epi_op_t ops[FUSEML_MAX_EPI_OPS];
  const int n = fuse_diamonds(desc->ops, desc->n_ops, ops);
  for (int i = 0; i < n; ++i) {
    const int32_t oc = ops[i].opcode;
    if (oc == FUSEML_OP_SAVE || oc == FUSEML_OP_SWAP || oc == FUSEML_OP_ADD_SAVED || oc == FUSEML_OP_MUL_SAVED) return true;
  }
  return false;
}

int32_t fuseml_sm100_schedule(const fuseml_gemm_desc_t* desc, const fuseml_plan_t* plan_in, int32_t unit,
                              fuseml_work_item_t* items, int32_t max_items, int32_t* n_units) {
  if (plan_in == nullptr || (items == nullptr && max_items > 0)) return -FUSEML_E_NULL;
  int rc = validate_desc(desc);
  if (rc != FUSEML_OK) return -rc;
  rc = check_plan(plan_in);
  if (rc != FUSEML_OK) return -rc;
  // the geometry of fuseml_sm100_gemm_epilogue
  const bool f32 = desc->ab_dtype == FUSEML_F32;
  const int64_t K = f32 ? 3 * desc->K : desc->K;
  const int BK = f32 ? 32 : 64;
  const int CGr = plan_in->cluster;
  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.tiles_m = static_cast<int32_t>((desc->M + kTileM * CGr - 1) / (kTileM * CGr));
  p.tiles_n = static_cast<int32_t>((desc->N + plan_in->tile_n - 1) / plan_in->tile_n);
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.num_kb = static_cast<int32_t>((K + BK - 1) / BK);
  p.red_kinds = desc->reduce.kinds;
  p.group_m = (plan_in->flags & FUSEML_PLAN_GROUP_N) ? -std::min(plan_in->group_m, p.tiles_n) : std::min(plan_in->group_m, p.tiles_m);
  int32_t units;
  if (plan_in->split_k > 1) {
    p.kb_per_split = (p.num_kb + plan_in->split_k - 1) / plan_in->split_k;
    p.split_k = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;
    units = p.num_tiles * p.split_k;
  } else if ((plan_in->flags & FUSEML_PLAN_STREAM_K) && !program_uses_saved(desc)) {
    p.stream_k = 1;
    units = plan_in->grid / CGr;
  } else {
    units = std::min(plan_in->grid, p.num_tiles * CGr) / CGr;
  }
  if (n_units != nullptr) *n_units = units;
  if (units < 1 || unit < 0 || unit >= units) return -FUSEML_E_PLAN;
  WorkWalk walk;
  walk.init(p, unit, units);
  WorkItem w;
  int32_t n = 0;
  while (walk.next(&w)) {
    if (n < max_items) {
      int32_t tm, tn;
      tile_coords(w.tile, p.tiles_m, p.tiles_n, p.group_m, &tm, &tn);
      items[n] = fuseml_work_item_t{w.tile, w.kb0, w.kb1, w.kind, w.after, w.slot, tm, tn};
    }
    ++n;
  }
  return n;
}

int fuseml_sm100_gemm_epilogue_noalloc(const fuseml_gemm_desc_t* desc, const fuseml_plan_t* plan_in,
                                       void* cuda_stream) {
  int rc = validate_desc(desc);
  if (rc != FUSEML_OK) return rc;
  fuseml_plan_t plan;
  if (plan_in != nullptr) {
    plan = *plan_in;
  } else {
    fuseml_device_props_t props;
    if (fuseml_sm100_query(&props) != FUSEML_OK) return FUSEML_E_DEVICE;
    // a plan made here never splits K: the partial tiles would eat the fixed scratch budget
    rc = make_plan(desc, &props, &plan, /*allow_split_k=*/false);
    if (rc != FUSEML_OK) return rc;
  }
  rc = check_plan(&plan);
  if (rc != FUSEML_OK) return rc;
  if (plan.split_k < 1) plan.split_k = 1;
  WorkspaceLayout w;
  workspace_layout(desc, &plan, &w);
  if (w.total > kNoAllocScratchBytes) return FUSEML_E_LIMIT;
  void* scratch = nullptr;
  rc = noalloc_scratch_address(&scratch);
  if (rc != FUSEML_OK) return rc;
  fuseml_gemm_desc_t local = *desc;       // the caller's descriptor is left untouched
  local.reduce.workspace = scratch;
  local.reduce.workspace_bytes = kNoAllocScratchBytes;
  return fuseml_sm100_gemm_epilogue(&local, &plan, cuda_stream);
}

int fuseml_sm100_set_diagnostics(int64_t wait_limit_us, int32_t drop_last_load) {
  if (wait_limit_us < 0 || wait_limit_us > 0xffffffffll) return FUSEML_E_LIMIT;
  g_diag_wait_limit_us.store(static_cast<uint32_t>(wait_limit_us), std::memory_order_relaxed);
  g_diag_drop_last_load.store(drop_last_load ? 1 : 0, std::memory_order_relaxed);
  return FUSEML_OK;
}

int fuseml_sm100_device_status(void* cuda_stream, int32_t* status_out) {
  if (status_out == nullptr) return FUSEML_E_NULL;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
  int32_t v = 0;
  if (cudaMemcpyFromSymbolAsync(&v, g_status_word, sizeof(v), 0, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
      cudaStreamSynchronize(stream) != cudaSuccess) {
    cudaGetLastError();
    return FUSEML_E_LAUNCH;
  }
  *status_out = v;
  if (v != 0) {
    const int32_t zero = 0;
    cudaMemcpyToSymbolAsync(g_status_word, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, stream);
    cudaStreamSynchronize(stream);
    return FUSEML_E_TIMEOUT;
  }
  return FUSEML_OK;
}

#ifdef FUSEML_STALL_COUNTERS
// diagnostic builds only: copy the per-CTA stall counters of the last launches to the host
int fuseml_debug_stalls(unsigned long long* out, int ctas) {
  if (ctas > 1024) ctas = 1024;
  return cudaMemcpyFromSymbol(out, fuseml::v2::g_stall, sizeof(unsigned long long) * 16 * ctas) == cudaSuccess ? 0 : 1;
}
#endif

}  // extern "C"
