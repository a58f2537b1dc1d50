// One pre-norm block (norm, q/k/v, rotation and cache write, attention, output projection, norm,
// gated feed-forward) enqueued by ONE call from the host language.
//
// A step that is not replayed from a CUDA graph (a prompt portion, a mixed batch) is enqueued kernel
// by kernel; done from Python that costs about 150 us per layer (eight calls into this library, ten
// allocations, the checks between them), which bounds every step of fewer than about a thousand
// tokens at small layer sizes.  This file holds the same sequence as host code: the choice of kernel
// by row count and shape that ops.py makes for each product (few rows / small / many rows; K slices
// left to the consumer), for q/k/v (rotation in the product's epilogue, slices added by the rotation
// kernel, or product then rotation) and for attention (merged into the output projection for small
// decode batches, or attention then projection), and the calls into the kernels' own entry points.
// The thresholds come from the caller (they are ops.py's, which stays the one place that sets
// them); a shape that ops.py would hand to a kernel this file does not call is answered with
// CO_BLOCK_UNSUPPORTED before anything is launched, and the caller runs its own sequence.
//
// Temporaries live in one scratch area that the caller provides (its size is asked for with
// dry_run = 1); the block's output (bfloat16 [T, H], or a float32 stack of partial sums
// [splits, T, H] that the next norm adds) goes where the caller says, its kind being part of the plan.
#include "common.cuh"

#include <cstdint>

extern "C" {
int coheryn_add_rmsnorm(float* resid, const void* delta, int delta_dtype, const int* rows, const void* weight, int wdtype,
                        float eps, void* out, int out_dtype, int n_rows, int H, int update, cudaStream_t stream);
int coheryn_add_parts_rmsnorm(float* resid, const float* parts, int splits, long split_stride, const int* rows,
                              const void* weight, int wdtype, float eps, void* out, int out_dtype, int n_rows, int H,
                              int update, cudaStream_t stream);
int coheryn_rope_kv_write_parts(const float* parts, int splits, long split_stride, const void* bias, int bias_dtype,
                                void* q_out, const int* positions, const float* cos_sin, const int* slots, void* k_cache,
                                void* v_cache, int T, int nh, int nkv, int hd, int page_size, cudaStream_t stream);
int coheryn_rope_kv_write(void* qkv, int dtype, const int* positions, const float* cos_sin, const int* slots, void* k_cache,
                          void* v_cache, int T, int nh, int nkv, int hd, int rot, int page_size, int write_kv,
                          cudaStream_t stream);
int coheryn_gemm_bf16_small(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype, int M,
                            int N, int K, long ldx, long ldo, int epilogue, cudaStream_t stream);
int coheryn_qkv_rope_bf16_small(const void* x, const void* w, const void* bias, int bias_dtype, void* q_out, long ldq,
                                const int* positions, const float* cos_sin, const int* slots, void* k_cache, void* v_cache,
                                int M, int K, long ldx, int nh, int nkv, int hd, int page_size, cudaStream_t stream);
long coheryn_gemm_tc_workspace_floats(int M, int N, int K);
int coheryn_gemm_bf16_tc(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype, int M,
                         int N, int K, long ldx, long ldo, int epilogue, int* status, float* workspace,
                         long workspace_floats, cudaStream_t stream);
int coheryn_gemm_tc_parts_count(int M, int N, int K);
int coheryn_gemm_bf16_tc_parts(const void* x, const void* w, float* parts, int M, int N, int K, long ldx, int* status,
                               cudaStream_t stream);
int coheryn_gemm_tc_few_splits(int N, int K);
int coheryn_gemm_bf16_tc_few(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype, int M,
                             int N, int K, long ldx, long ldo, int epilogue, int* status, float* workspace,
                             long workspace_floats, int defer, cudaStream_t stream);
}

// Entry points of the attention library of the layer's head size (a library of its own).
typedef int (*co_attention_fn)(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                               const void* v_cache, const int* block_tables, int max_blocks, const int* cu_q,
                               const int* kv_lens, int B, int nh, int nkv, int page_size, int window, float scale,
                               int max_rows, int any_small, int any_large, int max_kv_len, float* scratch,
                               long scratch_floats, int* status, int total_tokens, int num_pages, int settled,
                               cudaStream_t stream);
typedef int (*co_attention_oproj_fn)(const void* q, long q_stride, const void* k_cache, const void* v_cache,
                                     const int* block_tables, int max_blocks, const int* cu_q, const int* kv_lens, int B,
                                     int nh, int nkv, int page_size, int window, float scale, int max_kv_len,
                                     float* scratch, long scratch_floats, const void* w, long ldw, int H, const void* bias,
                                     int bias_dtype, float* parts, int settled, cudaStream_t stream);
typedef long (*co_attn_scratch_fn)(int B, int nkv, int max_kv_len);

// What a layer is made of: constant from the moment its weights are bound.
struct CoBlockLayer {
  const void* norm1_w; const void* norm2_w;
  const void* w_qkv; const void* b_qkv;
  const void* w_o; const void* b_o;
  const void* w_gate_up; const void* w_down;
  const float* cos_sin;
  co_attention_fn attention; co_attention_oproj_fn attention_oproj; co_attn_scratch_fn attn_scratch_floats;
  float eps1, eps2, scale;
  int norm1_wdtype, norm2_wdtype, b_qkv_dtype, b_o_dtype;
  int H, nh, nkv, hd, I, rot, window, gated_code;
  int mixer_partial, ff_partial;      // the part may hand partial sums to the next norm
};

// What a step is: the same for every layer of the step.
struct CoBlockStep {
  const int* positions; const int* cu_q; const int* kv_lens;
  int* tc_status;
  cudaStream_t stream;
  int T, B, min_q_len, max_q_len, max_kv_len, settled;
};

// ops.py's thresholds, as they stand when the step is run.
struct CoBlockTuning {
  long small_weight_elements, few_large_weight, attn_oproj_merge_bytes;
  int few_m, few_defer_m, few_head_m, small_m, small_m_short, defer_min_k, defer_min_k_wide;
  int qkv_rope_m, qkv_parts_m, qkv_parts_few_from, attn_oproj_m;
};

// What the block's output is: kind 1 = bfloat16 [T, H]; 2 = float32 [splits, T, H].
// The rest says which way each step of the block goes (tests compare it with ops.py's predicates):
// qkv_route 1 = rotation in the product's epilogue, 2 = K slices of the few-rows product added by the
// rotation kernel, 3 = those of the many-rows product, 4 = product (qkv_linear) then rotation; merged = 1
// when attention is merged into the output projection, else o_route; the products' routes are
// 1 few rows, 2 few rows with the K slices left to the consumer, 3 small, 4 many rows.
struct CoBlockPlan {
  long scratch_bytes;
  int out_kind, out_splits;
  int qkv_route, qkv_parts, qkv_linear, merged, o_route, gate_route, down_route;
};

#define CO_BLOCK_UNSUPPORTED 3    // nothing was launched: run the parts one by one
#define CO_BLOCK_ATTENTION_FAILED 2   // the message is the attention library's

namespace {

enum Route { R_NONE = 0, R_FEW, R_FEW_DEFER, R_SMALL, R_TC };

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

struct Router {
  const CoBlockTuning& t;
  bool operands_ok(int K, long ldx, const void* x, const void* w) const {
    return K % 8 == 0 && ldx % 8 == 0 && aligned16(x) && aligned16(w);
  }
  bool few_shape_ok(int M, int K, long ldx, const void* x, const void* w, int limit) const {
    return 0 < M && M <= limit && operands_ok(K, ldx, x, w);
  }
  bool few_ok(int M, int N, int K, long ldx, const void* x, const void* w) const {
    const int limit = (long)N * K >= t.few_large_weight ? t.few_head_m : t.few_m;
    return few_shape_ok(M, K, ldx, x, w, limit) && coheryn_gemm_tc_few_splits(N, K) == 1;
  }
  bool small_ok(int M, int N, int K, long ldx, const void* x, const void* w) const {
    return ((0 < M && M <= t.small_m) || (0 < M && M <= t.small_m_short && (long)N * K <= t.small_weight_elements)) &&
           operands_ok(K, ldx, x, w);
  }
  bool tc_ok(int M, int K, long ldx, const void* x, const void* w) const {
    return M > t.small_m && operands_ok(K, ldx, x, w);
  }
  // ops.linear: the route of y = x w^T and, for R_FEW_DEFER, the number of K slices.
  Route linear(int M, int N, int K, long ldx, const void* x, const void* w, bool partial_ok, int* splits) const {
    *splits = 1;
    if (partial_ok && M > 0 && K >= (M > t.small_m_short ? t.defer_min_k_wide : t.defer_min_k) &&
        few_shape_ok(M, K, ldx, x, w, t.few_defer_m)) {
      const int s = coheryn_gemm_tc_few_splits(N, K);
      if (s > 1) {
        *splits = s;
        return R_FEW_DEFER;
      }
    }
    if (few_ok(M, N, K, ldx, x, w)) return R_FEW;
    if (small_ok(M, N, K, ldx, x, w)) return R_SMALL;
    if (tc_ok(M, K, ldx, x, w)) return R_TC;
    return R_NONE;
  }
};

struct Arena {
  char* base;
  size_t off;
  void* workspace = nullptr;      // one area for the K slices of whichever many-rows product is running
  long workspace_floats = 0;
  void* take(size_t bytes) {
    off = (off + 255) & ~(size_t)255;
    void* p = base ? (void*)(base + off) : nullptr;
    off += bytes;
    return p;
  }
};

}  // namespace

namespace {

struct BlockIo {
  void* k_cache; void* v_cache; int num_pages, page_size;
  const int* block_tables; int max_blocks; const int* slots;
  float* resid; const void* delta; int delta_kind, delta_splits;
  void* out;
};

#define RUN(call)                      \
  do {                                 \
    if (launch) {                      \
      const int rc__ = (call);         \
      if (rc__) return rc__;           \
    }                                  \
  } while (0)
#define RUN_ATTENTION(call)                              \
  do {                                                   \
    if (launch && (call)) return CO_BLOCK_ATTENTION_FAILED; \
  } while (0)

// y = x w^T (+ bias) by the route chosen; `out` is [M, N] of out_dtype (or [M, N / 2] with a gated
// epilogue), or the float32 stack of K slices for R_FEW_DEFER.
int run_linear(Route route, Arena& A, bool launch, const CoBlockStep& S, const void* x, long ldx, const void* w,
               const void* bias, int bias_dtype, void* out, int M, int N, int K, long ldo, int epilogue) {
  const int bd = bias ? bias_dtype : CO_F32;
  switch (route) {
    case R_FEW:
      RUN(coheryn_gemm_bf16_tc_few(x, w, bias, bd, out, CO_BF16, M, N, K, ldx, ldo, epilogue, S.tc_status, nullptr, 0, 0,
                                   S.stream));
      return 0;
    case R_FEW_DEFER:
      RUN(coheryn_gemm_bf16_tc_few(x, w, bias, bd, out, CO_F32, M, N, K, ldx, N, 0, S.tc_status, nullptr, 0, 1, S.stream));
      return 0;
    case R_SMALL:
      RUN(coheryn_gemm_bf16_small(x, w, bias, bd, out, CO_BF16, M, N, K, ldx, ldo, epilogue, S.stream));
      return 0;
    case R_TC: {
      const long floats = coheryn_gemm_tc_workspace_floats(M, N, K);     // > 0: K is split
      float* ws = floats ? (float*)A.workspace : nullptr;      // the kernel that adds the slices follows in the same call
      if (floats > A.workspace_floats) return CO_BLOCK_UNSUPPORTED;
      RUN(coheryn_gemm_bf16_tc(x, w, bias, bd, out, CO_BF16, M, N, K, ldx, ldo, epilogue, S.tc_status, ws, floats,
                               S.stream));
      return 0;
    }
    default:
      return CO_BLOCK_UNSUPPORTED;
  }
}

int block_pass(const CoBlockLayer& L, const CoBlockStep& S, const CoBlockTuning& tn, const BlockIo& io, char* scratch,
               bool launch, CoBlockPlan* plan) {
  const int T = S.T, B = S.B, H = L.H, I = L.I, nh = L.nh, nkv = L.nkv, hd = L.hd;
  if (T <= 0 || B <= 0 || nkv <= 0 || nh % nkv || S.max_kv_len <= 0 || S.min_q_len <= 0) return CO_BLOCK_UNSUPPORTED;
  const int Nq = nh * hd, Nqkv = (nh + 2 * nkv) * hd, G = nh / nkv;
  const Router R{tn};
  Arena A{scratch, 0};
  cudaStream_t stream = S.stream;

  // The many-rows product adds its K slices with a kernel of its own before the next product starts:
  // the four products share one area for them.
  {
    long f = coheryn_gemm_tc_workspace_floats(T, Nqkv, H);
    const long f2 = coheryn_gemm_tc_workspace_floats(T, H, Nq), f3 = coheryn_gemm_tc_workspace_floats(T, 2 * I, H),
               f4 = coheryn_gemm_tc_workspace_floats(T, H, I);
    f = f > f2 ? f : f2;
    f = f > f3 ? f : f3;
    f = f > f4 ? f : f4;
    A.workspace_floats = f;
    A.workspace = f ? A.take((size_t)f * 4) : nullptr;
  }

  // x^ = norm(residual += delta)
  void* xn = A.take((size_t)T * H * 2);
  if (io.delta_kind == 2)
    RUN(coheryn_add_parts_rmsnorm(io.resid, (const float*)io.delta, io.delta_splits, (long)T * H, nullptr, L.norm1_w,
                                  L.norm1_wdtype, L.eps1, xn, CO_BF16, T, H, 1, stream));
  else
    RUN(coheryn_add_rmsnorm(io.resid, io.delta_kind == 1 ? io.delta : nullptr, io.delta_kind == 1 ? CO_BF16 : CO_F32,
                            nullptr, L.norm1_w, L.norm1_wdtype, L.eps1, xn, CO_BF16, T, H, io.delta_kind == 1 ? 1 : 0,
                            stream));

  // q, k, v; rotation; keys and values into the cache
  const void* q;
  long q_stride;
  const bool whole_head = L.rot == hd && hd % 16 == 0 && R.operands_ok(H, H, xn, L.w_qkv);
  plan->qkv_parts = 0;
  plan->qkv_linear = R_NONE;
  plan->o_route = R_NONE;
  if (whole_head && T <= tn.qkv_rope_m) {
    plan->qkv_route = 1;
    void* qb = A.take((size_t)T * Nq * 2);
    RUN(coheryn_qkv_rope_bf16_small(xn, L.w_qkv, L.b_qkv, L.b_qkv ? L.b_qkv_dtype : CO_F32, qb, Nq, S.positions, L.cos_sin,
                                    io.slots, io.k_cache, io.v_cache, T, H, H, nh, nkv, hd, io.page_size, stream));
    q = qb;
    q_stride = Nq;
  } else {
    int count = 0;
    if (whole_head && tn.qkv_rope_m < T && T <= tn.qkv_parts_m) {
      const int few = coheryn_gemm_tc_few_splits(Nqkv, H);
      count = (few > 1 && tn.qkv_parts_few_from < T && T <= tn.few_defer_m) ? few : coheryn_gemm_tc_parts_count(T, Nqkv, H);
    }
    plan->qkv_parts = count > 1 ? count : 0;
    plan->qkv_route = count > 1 ? (count == coheryn_gemm_tc_few_splits(Nqkv, H) ? 2 : 3) : 4;
    if (count > 1) {
      float* parts = (float*)A.take((size_t)count * T * Nqkv * 4);
      if (count == coheryn_gemm_tc_few_splits(Nqkv, H))
        RUN(coheryn_gemm_bf16_tc_few(xn, L.w_qkv, nullptr, CO_F32, parts, CO_F32, T, Nqkv, H, H, Nqkv, 0, S.tc_status,
                                     nullptr, 0, 1, stream));
      else
        RUN(coheryn_gemm_bf16_tc_parts(xn, L.w_qkv, parts, T, Nqkv, H, H, S.tc_status, stream));
      void* qb = A.take((size_t)T * Nq * 2);
      RUN(coheryn_rope_kv_write_parts(parts, count, (long)T * Nqkv, L.b_qkv, L.b_qkv ? L.b_qkv_dtype : CO_F32, qb,
                                      S.positions, L.cos_sin, io.slots, io.k_cache, io.v_cache, T, nh, nkv, hd,
                                      io.page_size, stream));
      q = qb;
      q_stride = Nq;
    } else {
      void* qkv = A.take((size_t)T * Nqkv * 2);
      int splits;
      const Route r = R.linear(T, Nqkv, H, H, xn, L.w_qkv, false, &splits);
      plan->qkv_linear = r;
      const int rc = run_linear(r, A, launch, S, xn, H, L.w_qkv, L.b_qkv, L.b_qkv_dtype, qkv, T, Nqkv, H, Nqkv, 0);
      if (rc) return rc;
      RUN(coheryn_rope_kv_write(qkv, CO_BF16, S.positions, L.cos_sin, io.slots, io.k_cache, io.v_cache, T, nh, nkv, hd,
                                L.rot, io.page_size, 1, stream));
      q = qkv;
      q_stride = Nqkv;
    }
  }

  // attention over the cache and the output projection
  if (!(hd % 16 == 0 && 16 <= hd && hd <= 256 && q_stride % 8 == 0)) return CO_BLOCK_UNSUPPORTED;
  const void* mixed;
  int mixed_kind, mixed_splits = 1;
  const long tiles = (H + 127) / 128;
  const long merge_bytes = tiles * nh * B * ((S.max_kv_len + 127) / 128) * hd * 4;
  const bool merged = L.mixer_partial && S.max_q_len == 1 && merge_bytes <= tn.attn_oproj_merge_bytes &&
                      B <= (tn.attn_oproj_m < 16 ? tn.attn_oproj_m : 16) && T == B && G <= 16 &&
                      (S.max_kv_len + 127) / 128 + 1 <= 512 && aligned16(q) && Nq % 8 == 0 && aligned16(L.w_o) && H % 4 == 0;
  plan->merged = merged ? 1 : 0;
  if (merged) {
    const long floats = L.attn_scratch_floats(B, nkv, S.max_kv_len);
    float* as = (float*)A.take((size_t)floats * 4);
    float* parts = (float*)A.take((size_t)nh * B * H * 4);
    RUN_ATTENTION(L.attention_oproj(q, q_stride, io.k_cache, io.v_cache, io.block_tables, io.max_blocks, S.cu_q, S.kv_lens,
                                    B, nh, nkv, io.page_size, L.window, L.scale, S.max_kv_len, as, floats, L.w_o, Nq, H,
                                    L.b_o, L.b_o ? L.b_o_dtype : CO_F32, parts, S.settled, stream));
    mixed = parts;
    mixed_kind = 2;
    mixed_splits = nh;
  } else {
    if (Nq % 4) return CO_BLOCK_UNSUPPORTED;
    const int max_rows = S.max_q_len * G;
    const int any_small = S.min_q_len * G <= 16, any_large = max_rows > 16;
    long floats = 0;
    float* as = nullptr;
    if (any_small && G <= 16) {
      floats = L.attn_scratch_floats(B, nkv, S.max_kv_len);
      as = (float*)A.take((size_t)floats * 4);
    }
    void* o = A.take((size_t)T * Nq * 2);
    RUN_ATTENTION(L.attention(q, q_stride, o, Nq, io.k_cache, io.v_cache, io.block_tables, io.max_blocks, S.cu_q, S.kv_lens,
                              B, nh, nkv, io.page_size, L.window, L.scale, max_rows, any_small, any_large, S.max_kv_len, as,
                              floats, S.tc_status, T, io.num_pages, S.settled, stream));
    const Route r = R.linear(T, H, Nq, Nq, o, L.w_o, L.mixer_partial != 0, &mixed_splits);
    plan->o_route = r;
    mixed_kind = r == R_FEW_DEFER ? 2 : 1;
    void* mb = A.take(mixed_kind == 2 ? (size_t)mixed_splits * T * H * 4 : (size_t)T * H * 2);
    const int rc = run_linear(r, A, launch, S, o, Nq, L.w_o, L.b_o, L.b_o_dtype, mb, T, H, Nq, H, 0);
    if (rc) return rc;
    mixed = mb;
  }

  // x^ = norm(residual += mixer output), where the first one was: the q/k/v product has consumed that
  void* xn2 = xn;
  if (mixed_kind == 2)
    RUN(coheryn_add_parts_rmsnorm(io.resid, (const float*)mixed, mixed_splits, (long)T * H, nullptr, L.norm2_w,
                                  L.norm2_wdtype, L.eps2, xn2, CO_BF16, T, H, 1, stream));
  else
    RUN(coheryn_add_rmsnorm(io.resid, mixed, CO_BF16, nullptr, L.norm2_w, L.norm2_wdtype, L.eps2, xn2, CO_BF16, T, H, 1,
                            stream));

  // act(gate) * up, then down
  void* act = A.take((size_t)T * I * 2);
  Route gr = R_NONE;
  if (R.few_ok(T, 2 * I, H, H, xn2, L.w_gate_up)) gr = R_FEW;
  else if (R.small_ok(T, 2 * I, H, H, xn2, L.w_gate_up)) gr = R_SMALL;
  else if (R.tc_ok(T, H, H, xn2, L.w_gate_up)) gr = R_TC;
  plan->gate_route = gr;
  int rc = run_linear(gr, A, launch, S, xn2, H, L.w_gate_up, nullptr, CO_F32, act, T, 2 * I, H, I, L.gated_code);
  if (rc) return rc;
  int out_splits;
  const Route dr = R.linear(T, H, I, I, act, L.w_down, L.ff_partial != 0, &out_splits);
  plan->down_route = dr;
  rc = run_linear(dr, A, launch, S, act, I, L.w_down, nullptr, CO_F32, io.out, T, H, I, H, 0);
  if (rc) return rc;
  plan->out_kind = dr == R_FEW_DEFER ? 2 : 1;
  plan->out_splits = out_splits;
  plan->scratch_bytes = (long)A.off + 256;
  return 0;
}

}  // namespace

// Runs (or, with dry_run, only plans) one block.  Returns 0, 1 (an error of this library: see
// coheryn_last_error), CO_BLOCK_ATTENTION_FAILED (an error of the attention library) or
// CO_BLOCK_UNSUPPORTED (nothing launched).  `plan` always receives the output's kind and the scratch
// bytes the block needs; a run checks both against what it was given before it launches anything.
CO_EXPORT int coheryn_prenorm_block_bf16(const CoBlockLayer* layer, const CoBlockStep* step, const CoBlockTuning* tuning,
                                         void* k_cache, void* v_cache, int num_pages, int page_size,
                                         const int* block_tables, int max_blocks, const int* slots, float* resid,
                                         const void* delta, int delta_kind, int delta_splits, void* out, int out_kind,
                                         int out_splits, void* scratch, long scratch_bytes, int dry_run,
                                         CoBlockPlan* plan) {
  if (!layer || !step || !tuning || !plan) CO_FAIL("prenorm_block: a description is missing");
  if (!layer->attention || !layer->attention_oproj || !layer->attn_scratch_floats)
    CO_FAIL("prenorm_block: the attention library's entry points are missing");
  const BlockIo io{k_cache, v_cache, num_pages, page_size, block_tables, max_blocks, slots,
                   resid,   delta,   delta_kind, delta_splits, out};
  int rc = block_pass(*layer, *step, *tuning, io, nullptr, false, plan);
  if (rc || dry_run) return rc;
  if (plan->out_kind != out_kind || (out_kind == 2 && plan->out_splits != out_splits))
    CO_FAIL("prenorm_block: the output was prepared as kind %d with %d parts, the plan says %d with %d", out_kind,
            out_splits, plan->out_kind, plan->out_splits);
  if (!scratch || scratch_bytes < plan->scratch_bytes || ((uintptr_t)scratch & 255))
    CO_FAIL("prenorm_block: %ld bytes of scratch (256-byte aligned) are needed, %ld were given", plan->scratch_bytes,
            scratch_bytes);
  if (!resid || !out || !k_cache || !v_cache || !block_tables || !slots) CO_FAIL("prenorm_block: a buffer is missing");
  CoBlockPlan again;
  return block_pass(*layer, *step, *tuning, io, (char*)scratch, true, &again);
}
