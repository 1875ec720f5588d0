// Host-only part of the C ABI: descriptor validation, the roofline router that
// picks tile / stage / cluster shapes, and the workspace arithmetic.  No CUDA
// call is made here, so these functions work (and are tested) on a machine
// without a GPU.
//
// The router replaces the reference's three-tier cost model
// (fuseml/passes/topology.py:479-571: penalty-vs-savings with per-arch tables;
// fuseml/passes/fusion_pass.py:463-498: the M*N < 500000 "tiny" bypass;
// fuseml/codegen/cublas_epilogue.py:166-258: the cuBLAS Lt pattern match) and the
// analytic SRAM autotuner (fuseml/codegen/sram_autotuner.py:135-213, 336-437).
// There is a single tier here - the fused sm_100a kernel - so the router only
// decides *how* to run it and predicts the time from the roofline.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>

#include "host_plan.h"

namespace fuseml {

int dtype_bytes(int32_t dt) {
  switch (dt) {
    case FUSEML_BF16:
    case FUSEML_F16:
      return 2;
    case FUSEML_F32:
      return 4;
    default:
      return 0;
  }
}

void default_props(fuseml_device_props_t* p) {
  p->sm_count = 148;
  p->cc_major = 10;
  p->cc_minor = 0;
  p->smem_per_block_optin = 232448;  // 227 KB
  p->tmem_cols = 512;
  p->l2_bytes = 126 * 1024 * 1024;
  p->hbm_gbs = 7700.0;               // HGX B200 HBM3e
  p->tensor_tflops = 2250.0;         // dense bf16
}

static bool op_uses_operand(int32_t opcode) {
  return opcode == FUSEML_OP_ADD_T || opcode == FUSEML_OP_MUL_T || opcode == FUSEML_OP_SUB_T ||
         opcode == FUSEML_OP_RSUB_T || opcode == FUSEML_OP_STORE_AUX || opcode == FUSEML_OP_GELU_ERF_BWD_T;
}

int a_layout(const fuseml_gemm_desc_t* d) {
  if (d->a_stride_k == 0 || d->a_stride_k == 1) return 0;
  if (d->lda != 1 && d->M > 1) return -1;
  if (d->ab_dtype == FUSEML_F32) return 1;                      // expanded by plain loads: any stride
  const int eb = dtype_bytes(d->ab_dtype);
  if (d->a_stride_k < d->M || (d->a_stride_k * eb) % 16 != 0) return -1;
  return b_layout(d) == 1 ? 1 : -1;                             // kernels exist for MN-major A with MN-major B only
}

int b_layout(const fuseml_gemm_desc_t* d) {
  const int eb = dtype_bytes(d->ab_dtype);
  const bool tma = d->ab_dtype != FUSEML_F32;
  if (d->b_stride_k == 1) {
    if (d->N == 1) return 0;
    if (d->b_stride_n >= d->K && (!tma || (d->b_stride_n * eb) % 16 == 0)) return 0;
  }
  if (d->b_stride_n == 1) {
    if (d->K == 1) return 1;
    if (d->b_stride_k >= d->N && (!tma || (d->b_stride_k * eb) % 16 == 0)) return 1;
  }
  return -1;
}

int validate_desc(const fuseml_gemm_desc_t* d) {
  if (d == nullptr) return FUSEML_E_NULL;
  if (d->a == nullptr || d->b == nullptr) return FUSEML_E_NULL;
  if (d->M <= 0 || d->N <= 0 || d->K <= 0) return FUSEML_E_SHAPE;
  if (d->M > 0x7fffff00ll || d->N > 0x7fffff00ll || d->K > 0x2a000000ll) return FUSEML_E_SHAPE;
  const int eb = dtype_bytes(d->ab_dtype);
  if (eb == 0) return FUSEML_E_DTYPE;
  if (dtype_bytes(d->out_dtype) == 0) return FUSEML_E_DTYPE;
  if (d->ab_dtype != FUSEML_F32) {
    // TMA reads A and B directly: 16-byte aligned base, leading stride a multiple of
    // 16 bytes.  (fp32 operands are first expanded by a plain-load kernel, so any
    // stride works there.)
    if ((reinterpret_cast<uintptr_t>(d->a) & 15u) != 0 || (reinterpret_cast<uintptr_t>(d->b) & 15u) != 0)
      return FUSEML_E_LAYOUT;
    if (d->a_stride_k <= 1 && d->M > 1 && (d->lda < d->K || (d->lda * eb) % 16 != 0)) return FUSEML_E_LAYOUT;
  } else if (d->a_stride_k <= 1 && d->M > 1 && d->lda < d->K) {
    return FUSEML_E_LAYOUT;
  }
  if (d->a_stride_k < 0) return FUSEML_E_LAYOUT;
  if (b_layout(d) < 0) return FUSEML_E_LAYOUT;
  if (a_layout(d) < 0) return FUSEML_E_LAYOUT;
  if (d->n_ops < 0 || d->n_ops > FUSEML_MAX_EPI_OPS) return FUSEML_E_EPILOGUE;
  if (d->n_operands < 0 || d->n_operands > FUSEML_MAX_OPERANDS) return FUSEML_E_EPILOGUE;
  for (int i = 0; i < d->n_ops; ++i) {
    const fuseml_epi_op_t& op = d->ops[i];
    if (op.opcode < 0 || op.opcode >= FUSEML_OP__COUNT) return FUSEML_E_EPILOGUE;
    if (op_uses_operand(op.opcode)) {
      if (op.slot < 0 || op.slot >= d->n_operands) return FUSEML_E_EPILOGUE;
      const fuseml_operand_t& o = d->operands[op.slot];
      if (o.ptr == nullptr) return FUSEML_E_NULL;
      if (dtype_bytes(o.dtype) == 0) return FUSEML_E_DTYPE;
      if (o.stride_m < 0 || o.stride_n < 0) return FUSEML_E_LAYOUT;
      if (op.opcode == FUSEML_OP_STORE_AUX && (o.stride_n != 1 || o.stride_m < d->N)) return FUSEML_E_LAYOUT;
    }
  }
  const fuseml_reduce_t& r = d->reduce;
  if (r.kinds != 0) {
    if (r.kinds & ~(FUSEML_RED_SUM | FUSEML_RED_MAX | FUSEML_RED_MEAN)) return FUSEML_E_REDUCTION;
    if (r.axis != FUSEML_AXIS_N && r.axis != FUSEML_AXIS_M && r.axis != FUSEML_AXIS_ALL)
      return FUSEML_E_REDUCTION;
    if ((r.kinds & FUSEML_RED_SUM) && r.out_sum == nullptr) return FUSEML_E_NULL;
    if ((r.kinds & FUSEML_RED_MAX) && r.out_max == nullptr) return FUSEML_E_NULL;
    if ((r.kinds & FUSEML_RED_MEAN) && r.out_mean == nullptr) return FUSEML_E_NULL;
  } else if (d->d == nullptr) {
    return FUSEML_E_NULL;  // nothing to produce
  }
  if (d->d != nullptr && d->ldd < d->N) return FUSEML_E_LAYOUT;
  return FUSEML_OK;
}

static int64_t round_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

int64_t split_ld(int64_t K) { return round_up(3 * K, 4); }

static double operand_bytes(const fuseml_gemm_desc_t* d) {
  double b = 0.0;
  bool seen[FUSEML_MAX_OPERANDS] = {false};
  for (int i = 0; i < d->n_ops; ++i) {
    const fuseml_epi_op_t& op = d->ops[i];
    if (!op_uses_operand(op.opcode) || op.slot < 0 || op.slot >= d->n_operands || seen[op.slot]) continue;
    seen[op.slot] = true;
    const fuseml_operand_t& o = d->operands[op.slot];
    const double rows = o.stride_m == 0 ? 1.0 : static_cast<double>(d->M);
    const double cols = o.stride_n == 0 ? 1.0 : static_cast<double>(d->N);
    b += rows * cols * dtype_bytes(o.dtype);
  }
  return b;
}

int make_plan(const fuseml_gemm_desc_t* d, const fuseml_device_props_t* props_in, fuseml_plan_t* plan,
              bool allow_split_k) {
  if (d == nullptr || plan == nullptr) return FUSEML_E_NULL;
  std::memset(plan, 0, sizeof(*plan));
  const int v = validate_desc(d);
  fuseml_device_props_t props;
  if (props_in) props = *props_in; else default_props(&props);

  const int eb = std::max(1, dtype_bytes(d->ab_dtype));
  const bool f32 = d->ab_dtype == FUSEML_F32;
  const double M = static_cast<double>(d->M), N = static_cast<double>(d->N), K = static_cast<double>(d->K);
  plan->flops = 2.0 * M * N * K;
  double bytes = M * K * eb + K * N * eb + operand_bytes(d);
  if (d->d != nullptr) bytes += M * N * std::max(1, dtype_bytes(d->out_dtype));
  if (d->reduce.kinds != 0) {
    const double len = d->reduce.axis == FUSEML_AXIS_N ? M : (d->reduce.axis == FUSEML_AXIS_M ? N : 1.0);
    int kinds = 0;
    for (int b = 1; b <= 4; b <<= 1) kinds += (d->reduce.kinds & b) ? 1 : 0;
    bytes += len * 4.0 * kinds;
  }
  plan->bytes = bytes;
  // fp32 operands run as three TF32 products (hi*hi + lo*hi + hi*lo): 3x the MMA work
  const double mma_flops = plan->flops * (f32 ? 3.0 : 1.0);
  const double tc_rate = props.tensor_tflops * (f32 ? 0.5 : 1.0);  // TF32 runs at half the bf16 rate
  plan->t_tensor_us = mma_flops / (tc_rate * 1e12) * 1e6;
  plan->t_hbm_us = bytes / (props.hbm_gbs * 1e9) * 1e6;

  plan->tile_m = 128;
  plan->tile_k = 128 / (f32 ? 4 : eb);
  plan->cluster = 1;
  plan->acc_stages = 2;

  // Candidate tile widths; pick the one with the smaller estimated time
  // (per-tile tensor time x waves, against the HBM time).
  int64_t tiles_m = (d->M + 127) / 128;
  const double per_sm_rate = tc_rate * 1e12 / std::max(1, props.sm_count);
  const int64_t k_eff = (f32 ? 3 : 1) * d->K;
  const int64_t k_pad = round_up(k_eff, plan->tile_k);
  double best = 1e300;
  int best_bn = 256;
  const int candidates[2] = {256, 128};
  for (int ci = 0; ci < 2; ++ci) {
    const int bn = candidates[ci];
    const int64_t tiles_n = (d->N + bn - 1) / bn;
    const int64_t tiles = tiles_m * tiles_n;
    const int64_t waves = (tiles + props.sm_count - 1) / props.sm_count;
    const double t_tile = 2.0 * 128.0 * bn * static_cast<double>(k_pad) / per_sm_rate * 1e6;
    // narrower tiles re-read A more often from L2 and keep the tensor pipe less busy per
    // shared-memory byte: a 5 % handicap keeps 256 the default when the wave counts tie
    const double t = std::max(waves * t_tile * (bn == 128 ? 1.05 : 1.0), plan->t_hbm_us);
    if (t < best) { best = t; best_bn = bn; }
  }
  // CTA pairs (cta_group::2): a 256 x 256 tile whose B operand is split between the two CTAs'
  // shared memories, so each SM ingests 32 KB instead of 48 KB per K block.  Measured on B200:
  // the pair kernel at full width beats both the single-CTA kernels and narrower pair tiles
  // (shaving the width to even out the last wave costs more in operand re-reads than the
  // wave saves), so it is used whenever there is more than one 128-row block and more than
  // 128 columns.  The kernels accept any multiple of 32 as tile width; the router does not
  // use that freedom yet.
  if (d->M > 128 && d->N > 128) {
    plan->cluster = 2;
    best_bn = 256;
    tiles_m = (d->M + 255) / 256;
    const int64_t tn = (d->N + 255) / 256;
    const int64_t units = std::max(1, props.sm_count / 2);
    const int64_t waves = (tiles_m * tn + units - 1) / units;
    best = std::max(waves * 2.0 * 256.0 * 256.0 * static_cast<double>(k_pad) / (2.0 * per_sm_rate) * 1e6,
                    plan->t_hbm_us);
  }
  // One row of tiles (M <= 128: decode-sized batches, small fp32 problems) and fewer tiles than
  // SMs: a 256-wide tile would leave most of the machine idle while a few CTAs walk the whole
  // K loop.  Narrow the tiles (multiples of 32 columns) until there is about one per SM: the
  // operand stream is then pulled by every SM, and each CTA's K loop issues proportionally
  // smaller MMAs.
  if (plan->cluster == 1 && tiles_m == 1 && d->N > 32) {
    const int64_t per_sm = (d->N + props.sm_count - 1) / std::max(1, props.sm_count);
    const int64_t width = std::min<int64_t>(256, std::max<int64_t>(32, round_up(per_sm, 32)));
    if (width < best_bn) best_bn = static_cast<int>(width);
  }
  // Split-K.  One K block costs a CTA about 570 cycles whatever the tile width (each MMA reads
  // its 128-row slice of A from shared memory), so a problem with one row of tiles and a long
  // K loop is bound by ceil(K/64) x 570 cycles per CTA however many SMs idle beside it.  Then
  // several CTAs share one full-width tile's K loop, each writes an fp32 partial tile to the
  // workspace, and a second kernel folds the partials in a fixed order and runs the epilogue.
  // Only without fused reductions, and only when the partial tiles (which cross L2 twice) are
  // small against what the split saves: at least 8 K blocks per CTA must disappear.
  plan->split_k = 1;
  if (allow_split_k && plan->cluster == 1 && tiles_m == 1 && d->reduce.kinds == 0 && d->d != nullptr) {
    const int64_t num_kb = k_pad / plan->tile_k;
    const int64_t wide_tiles = (d->N + 255) / 256;
    const int64_t max_split = std::min<int64_t>({props.sm_count / std::max<int64_t>(1, wide_tiles), num_kb / 4, 32});
    // the K loop of one CTA against the time the operands need to arrive from HBM anyway
    const double t_loop_us = static_cast<double>(num_kb) * 570.0 / 1900.0;
    const double t_floor_us = std::max(plan->t_hbm_us, 2.0);
    // measured on B200: the gain flattens once a CTA is left with about 8 K blocks (launch,
    // pipeline fill and the finish pass then dominate), so aim for that many per slice
    int64_t want = (num_kb + 7) / 8;
    want = std::min(want, max_split);
    if (want >= 2 && t_loop_us > 1.5 * t_floor_us && num_kb - num_kb / want >= 8) {
      // equal slices of ceil(num_kb / want) K blocks; drop the slices that would come out empty
      const int64_t per = (num_kb + want - 1) / want;
      plan->split_k = static_cast<int32_t>((num_kb + per - 1) / per);
      best_bn = d->N > 128 ? 256 : 128;
    }
  }
  plan->tile_n = best_bn;
  const int cg = plan->cluster;
  const int64_t tiles_n = (d->N + best_bn - 1) / best_bn;
  const int64_t tiles = tiles_m * tiles_n;
  const int64_t units = std::max(1, props.sm_count / cg);
  plan->grid = static_cast<int32_t>(std::min<int64_t>(tiles, units) * cg);
  if (plan->split_k > 1) plan->grid = static_cast<int32_t>(tiles * plan->split_k);   // one (tile, K slice) per CTA
  // K-split last wave of CTA-pair launches (the walk itself is WorkWalk in gemm_params.cuh): with
  // T tiles on U pairs the last wave holds R = T % U tiles.  R <= U / 2: each is cut into S = U / R
  // equal K slices, one per pair, and the wave takes 1/S of a tile's time; the later slices pass
  // through the workspace (256 KB per pair).  Chosen when the saving, (1 - 1/S) of a wave, is at
  // least 3 % of the launch and the slices stay long: measured on B200, 4096 x 4096 x 16384
  // (34 tiles left, 128 K blocks per slice) gains 10 %, 1024 x 16384 x 4096 (34 tiles left, 32 K
  // blocks per slice) loses 3 % to the pass of the partial accumulators through the workspace.
  // R > U / 2 (the idle pairs take the K tails of the others' tiles) is never chosen here: the
  // helpers' short parts and the owners' wait for them cost what the shorter wave saves
  // (2048 x 4096 x 16384, 54 tiles left: 198 us either way; 1024 x 4096 x 16384, 64 lone tiles:
  // 110 us against 99 us); a caller or the plan tuner may still set the flag.
  if (cg == 2 && plan->split_k == 1 && allow_split_k) {
    const int64_t rem = tiles % units;
    const int64_t waves = (tiles + units - 1) / units;
    const int64_t num_kb = k_pad / plan->tile_k;
    const int64_t slices = rem > 0 ? units / rem : 0;
    if (slices >= 2 && num_kb >= 64 * slices && (1.0 - 1.0 / static_cast<double>(slices)) / static_cast<double>(waves) >= 0.03) {
      plan->flags |= FUSEML_PLAN_STREAM_K;
      plan->grid = static_cast<int32_t>(units * cg);          // every pair takes part in the last wave
    }
  }
  // Rasterisation: tiles are walked in groups of group_m tile rows (all columns of one group
  // before the next group).  The group's rows of A stay in L2 while B streams past once per
  // group, so DRAM reads are about bytes(A) + ceil(tiles_m / group_m) * bytes(B): the taller the
  // group, the fewer passes over B, as long as the A slab (group_m * tile rows * K) still fits
  // beside the stream.  Measured on B200 with the kernel power-capped: cycle counts do not
  // depend on group_m, but the saved DRAM traffic returns as SM clock (8192 x 16384 x 4096:
  // group of 16 against 4, 3.7x less DRAM traffic, 8 % faster); slabs above a quarter of L2
  // lose again.  So: the largest power of two whose slab stays within 32 MiB.
  // With more tile rows than tile columns the same is done the other way round
  // (FUSEML_PLAN_GROUP_N): bands of group_m tile columns walked through all the tile rows, the
  // band's columns of B kept while A streams past once per band.  The groups are then longer
  // (more waves per group, fewer waves that straddle two groups and read the kept slabs of
  // both): 8192 x 4096 x 4096 with row reductions 214 -> 210 us, 16384 x 4096 x 8192 885 -> 871 us,
  // both held under the power cap.
  // With a long K even a few slabs exceed the bound and nothing is kept from wave to wave; what
  // counts then is what one wave of `units` tiles reads, g slabs of the kept operand plus
  // units / g of the other, least for a square wave: g is raised to the power of two below
  // sqrt(units * other slab / kept slab).  Measured (8192 x 4096 x 16384, 8.4 MB per slab, one
  // launch under ncu): groups of 4 tile rows read 2.1 GB in 789 us, groups of 8 tile rows 1.77 GB
  // in 770 us, bands of 8 tile columns 1.34 GB; the four-block stack of such GEMMs runs 3.4 %
  // faster under the power cap with the bands than with groups of 4 rows.
  {
    const double slab_per_tile_row = 128.0 * cg * static_cast<double>(k_pad) * (f32 ? 4 : eb);
    const double slab_per_tile_col = static_cast<double>(best_bn) * static_cast<double>(k_pad) * (f32 ? 4 : eb);
    const bool by_cols = tiles_m > tiles_n && tiles >= 2 * units;
    const double kept = by_cols ? slab_per_tile_col : slab_per_tile_row;
    const double other = by_cols ? slab_per_tile_row : slab_per_tile_col;
    const int64_t along = by_cols ? tiles_n : tiles_m;
    int64_t g = 1;
    while (g * 2 <= along && static_cast<double>(g * 2) * kept <= 32.0 * 1024 * 1024) g *= 2;
    int64_t gw = 1;
    while (gw * 2 <= along && static_cast<double>(gw * 2) * static_cast<double>(gw * 2) * kept <= static_cast<double>(units) * other) gw *= 2;
    if (g < gw && tiles >= 2 * units) g = gw;
    if (by_cols) plan->flags |= FUSEML_PLAN_GROUP_N;
    plan->group_m = static_cast<int32_t>(std::max<int64_t>(1, std::min<int64_t>(g, along)));
  }

  // Shared memory: ring of (A 16 KB + this CTA's share of B) stages under the opt-in budget.
  const int kernel_bn = best_bn > 128 ? 256 : 128;   // the instance that runs it
  const int stage_bytes = 128 * 128 + (kernel_bn / cg) * 128;
  const int fixed = 4 * kernel_bn * 2 * 4 /* column-reduction scratch */ + 4 * kernel_bn * 4 /* staged row vectors */ +
                    256 /* barriers */ + 1024 /* alignment */;
  int stages = (props.smem_per_block_optin - fixed) / stage_bytes;
  stages = std::max(2, std::min(stages, cg == 2 ? 6 : (kernel_bn == 256 ? 4 : 6)));
  plan->stages = stages;
  plan->smem_bytes = stages * stage_bytes + fixed;
  plan->tmem_cols = 2 * kernel_bn;

  const double launch_us = 3.0;
  plan->t_est_us = best + launch_us;
  // too few tiles to occupy the machine, or a run time comparable to a launch: neither
  // roofline applies, the kernel is bound by the latency of one tile's K loop
  if (plan->t_est_us < 2.0 * launch_us || tiles * 4 < props.sm_count) plan->bound = 2;
  else plan->bound = (plan->t_tensor_us >= plan->t_hbm_us) ? 1 : 0;
  plan->fuse = (v == FUSEML_OK) ? 1 : 0;
  return v;
}

static int64_t align256(int64_t x) { return round_up(x, 256); }

void workspace_layout(const fuseml_gemm_desc_t* d, const fuseml_plan_t* plan, WorkspaceLayout* w) {
  std::memset(w, 0, sizeof(*w));
  int64_t off = 0;
  if (d->ab_dtype == FUSEML_F32) {
    const int64_t ld = split_ld(d->K);
    w->split_a_off = off;
    off += align256(d->M * ld * 4);
    w->split_b_off = off;
    off += align256(d->N * ld * 4);
  }
  if (d->reduce.kinds != 0) {
    const int64_t tiles_m = (d->M + plan->tile_m - 1) / plan->tile_m;   // 128-row blocks
    const int64_t tiles_n = (d->N + plan->tile_n - 1) / plan->tile_n;
    int64_t partials, len;
    // per row: one partial per column tile and per epilogue warp sharing the row (two)
    if (d->reduce.axis == FUSEML_AXIS_N) { partials = tiles_n * 2; len = d->M; }
    else if (d->reduce.axis == FUSEML_AXIS_M) { partials = tiles_m; len = d->N; }
    else { partials = plan->grid; len = 1; }
    w->partials = partials;
    w->len = len;
    if (d->reduce.kinds & (FUSEML_RED_SUM | FUSEML_RED_MEAN)) {
      w->red_sum_off = off;
      off += align256(partials * len * 4);
    }
    if (d->reduce.kinds & FUSEML_RED_MAX) {
      w->red_max_off = off;
      off += align256(partials * len * 4);
    }
  }
  if (plan->split_k > 1) {
    w->splitk_off = off;
    // whole tiles (rows padded to 128, columns to the tile width): the kernels address them
    // piece-major, see splitk_finish.cuh
    const int64_t tiles = ((d->M + 127) / 128) * ((d->N + plan->tile_n - 1) / plan->tile_n);
    off += align256(static_cast<int64_t>(plan->split_k) * tiles * 128 * plan->tile_n * 4);
  }
  if (plan->flags & FUSEML_PLAN_STREAM_K) {
    const int64_t ctas = plan->grid;
    w->sk_ws_off = off;
    off += align256(ctas * 128 * 256 * 4);
    w->sk_flags_off = off;
    w->sk_flags_bytes = align256(ctas * 4);
    off += w->sk_flags_bytes;
  }
  w->total = off;
}

}  // namespace fuseml
