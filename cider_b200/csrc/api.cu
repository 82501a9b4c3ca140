// C ABI of libcider_b200: argument validation, kernel selection, error text.
// Mirrors the host-side launch logic of the reference's primitives
// (csrc/src/w8a8_primitive.mm:137-276, pergroup_primitive.mm:138-312,
// w4a8_primitive.mm:175-283) without any allocation or global scratch.
#include <atomic>
#include <cstring>

#include "common.cuh"

namespace cider {

namespace {
thread_local std::string t_last_error;
std::atomic<int> g_backend{0};
std::atomic<int> g_pdl{0};
constexpr int kMaxDevices = 64;
int g_sm_count[kMaxDevices] = {0};
}  // namespace

void set_error(const std::string &msg) { t_last_error = msg; }
int fail(int code, const std::string &msg) {
  t_last_error = msg;
  return code;
}
int check_cuda(cudaError_t e, const char *what) {
  if (e == cudaSuccess) return CIDER_OK;
  return fail(CIDER_E_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}
bool pdl_enabled() { return g_pdl.load(std::memory_order_relaxed) != 0; }
int current_device() {
  int d = 0;
  cudaGetDevice(&d);
  return d;
}
int sm_count(int device) {
  if (device < 0 || device >= kMaxDevices) device = 0;
  if (g_sm_count[device] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0)
      n = 148;
    g_sm_count[device] = n;
  }
  return g_sm_count[device];
}

namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Workspace {
  int8_t *a_q = nullptr;
  float *sa = nullptr;
  uint8_t *w_scratch = nullptr;  // W4A8: repacked rows (reference layout) / int8 copy (odd shapes)
  void *splitk = nullptr;  // per-channel linear at small M: int32 slabs of the split-K plan
};

// W4A8 shapes whose packed rows the tensor-core and streaming kernels expand themselves
// (whole 16-byte chunks of a row per 128 of K); other shapes go through an int8 copy or
// the plain kernel.
bool w4_rows_shape(int64_t K) { return K >= 128 && K % 32 == 0; }

// Weight scratch of the two W4A8 entries: the reference layout [K/2, N] is repacked into
// rows ([N, K/2], N*K/2 bytes) per call; rows need nothing, except shapes the row kernels do
// not take, which are expanded to int8 (N*K bytes).
size_t w4_scratch_bytes(int op, int64_t N, int64_t K) {
  if (op == CIDER_OP_W4A8) return w4_rows_shape(K) ? (size_t)N * (size_t)K / 2 : 0;
  if (op == CIDER_OP_W4A8_ROWS) return w4_rows_shape(K) ? 0 : (size_t)N * (size_t)K;
  if (op == CIDER_OP_W4A8_ROWS_INT8COPY) return (size_t)N * (size_t)K;
  return 0;
}

size_t workspace_bytes(int op, int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const bool w4 = op == CIDER_OP_W4A8 || op == CIDER_OP_W4A8_ROWS || op == CIDER_OP_W4A8_ROWS_INT8COPY;
  if (M == 1 && !w4) return 0;
  size_t b = align_up((size_t)M * (size_t)K, 256) + align_up((size_t)M * sizeof(float), 256);
  if (w4) b += align_up(w4_scratch_bytes(op, N, K), 256);
  if (op == CIDER_OP_PERCHANNEL) b += align_up(plan_splitk(M, N, K).bytes, 256);
  if (op == CIDER_OP_PERGROUP) b += align_up(plan_pg_splitk(M, N, K).bytes, 256);
  return b;
}

int carve(int op, void *ws, size_t ws_bytes, int64_t M, int64_t N, int64_t K, Workspace *out) {
  const size_t need = workspace_bytes(op, M, N, K);
  if (need == 0) return CIDER_OK;
  if (ws == nullptr || ws_bytes < need)
    return fail(CIDER_E_WORKSPACE, "workspace too small: need " + std::to_string(need) + " bytes, got " +
                                       std::to_string(ws ? ws_bytes : 0));
  if (reinterpret_cast<uintptr_t>(ws) & 255u)
    return fail(CIDER_E_ALIGNMENT, "workspace must be 256-byte aligned");
  uint8_t *p = static_cast<uint8_t *>(ws);
  out->a_q = reinterpret_cast<int8_t *>(p);
  p += align_up((size_t)M * (size_t)K, 256);
  out->sa = reinterpret_cast<float *>(p);
  p += align_up((size_t)M * sizeof(float), 256);
  if (w4_scratch_bytes(op, N, K) > 0) out->w_scratch = p;
  if (op == CIDER_OP_PERCHANNEL && plan_splitk(M, N, K).bytes > 0) out->splitk = p;
  if (op == CIDER_OP_PERGROUP && plan_pg_splitk(M, N, K).bytes > 0) out->splitk = p;
  return CIDER_OK;
}

int check_dims(const char *op, int64_t M, int64_t N, int64_t K) {
  if (M < 0 || N <= 0 || K <= 0)
    return fail(CIDER_E_INVALID, std::string(op) + ": need M >= 0, N > 0, K > 0 (got M=" + std::to_string(M) +
                                     " N=" + std::to_string(N) + " K=" + std::to_string(K) + ")");
  if (M > (int64_t)1 << 30 || N > (int64_t)1 << 30 || K > (int64_t)1 << 30)
    return fail(CIDER_E_INVALID, std::string(op) + ": dimension exceeds 2^30");
  return CIDER_OK;
}

int check_group(const char *op, int64_t K, int gs) {
  if (gs != 64 && gs != 128 && gs != 256)
    return fail(CIDER_E_SHAPE, std::string(op) + ": group_size must be 64, 128, or 256 (got " +
                                   std::to_string(gs) + ")");
  if (K % gs != 0)
    return fail(CIDER_E_SHAPE, std::string(op) + ": K=" + std::to_string(K) +
                                   " is not a multiple of group_size=" + std::to_string(gs));
  return CIDER_OK;
}

int check_dtype(const char *op, int dt) {
  if (dt != CIDER_F32 && dt != CIDER_F16)
    return fail(CIDER_E_INVALID, std::string(op) + ": scale_dtype must be CIDER_F32 or CIDER_F16");
  return CIDER_OK;
}

int run_gemm(const GemmArgs &g, cudaStream_t st) {
  const int backend = g_backend.load();
  const bool tc_ok = gemm_tc_eligible(g);
  if (backend == 2 && !tc_ok)
    return fail(CIDER_E_SHAPE, "tensor-core GEMM requested but the shape / alignment does not allow it");
  if (backend != 1 && tc_ok) return launch_gemm_tc(g, st);
  return launch_gemm_generic(g, st);
}

}  // namespace
}  // namespace cider

using namespace cider;

extern "C" {

int cider_version(void) { return 100; }

const char *cider_last_error(void) { return t_last_error.c_str(); }

int cider_device_supported(int device) {
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return major == 10 ? 1 : 0;
}

size_t cider_workspace_bytes(int op, int64_t M, int64_t N, int64_t K) {
  if (op != CIDER_OP_PERCHANNEL && op != CIDER_OP_PERGROUP && op != CIDER_OP_W4A8 && op != CIDER_OP_W4A8_ROWS &&
      op != CIDER_OP_W4A8_ROWS_INT8COPY)
    return 0;
  return workspace_bytes(op, M, N, K);
}

int cider_quantize_per_token(const void *x, int64_t M, int64_t K, int64_t ldx, void *q, float *scale,
                             void *stream) {
  if (M < 0 || K < 0) return fail(CIDER_E_INVALID, "quantize_per_token: negative size");
  if (M == 0) return CIDER_OK;
  if (!q && K > 0) return fail(CIDER_E_INVALID, "quantize_per_token: null output");
  if (!scale) return fail(CIDER_E_INVALID, "quantize_per_token: null scale");
  if (!x && K > 0) return fail(CIDER_E_INVALID, "quantize_per_token: null input");
  if (ldx < K) return fail(CIDER_E_INVALID, "quantize_per_token: ldx < K");
  if (M > (int64_t)1 << 30 || K > (int64_t)1 << 30)
    return fail(CIDER_E_INVALID, "quantize_per_token: dimension exceeds 2^30");
  if (reinterpret_cast<uintptr_t>(x) & 1u)
    return fail(CIDER_E_ALIGNMENT, "quantize_per_token: x must be 2-byte aligned");
  return launch_quantize_per_token(static_cast<const __half *>(x), M, K, ldx, static_cast<int8_t *>(q),
                                   scale, static_cast<cudaStream_t>(stream));
}

static int check_rows(const char *op, const void *x, int64_t M, int64_t K, int64_t ldx) {
  if (M < 0 || K <= 0) return fail(CIDER_E_INVALID, std::string(op) + ": need M >= 0, K > 0");
  if (ldx < K) return fail(CIDER_E_INVALID, std::string(op) + ": ldx < K");
  if (M > (int64_t)1 << 30 || K > (int64_t)1 << 30) return fail(CIDER_E_INVALID, std::string(op) + ": dimension exceeds 2^30");
  if (M > 0 && !x) return fail(CIDER_E_INVALID, std::string(op) + ": null input");
  if (reinterpret_cast<uintptr_t>(x) & 1u) return fail(CIDER_E_ALIGNMENT, std::string(op) + ": x must be 2-byte aligned");
  return CIDER_OK;
}

int cider_row_absmax(const void *x, int64_t M, int64_t K, int64_t ldx, float *amax, void *stream) {
  int rc = check_rows("row_absmax", x, M, K, ldx);
  if (rc) return rc;
  if (M == 0) return CIDER_OK;
  if (!amax) return fail(CIDER_E_INVALID, "row_absmax: null output");
  return launch_row_absmax(static_cast<const __half *>(x), M, K, ldx, amax, static_cast<cudaStream_t>(stream));
}

int cider_quantize_given_amax(const void *x, int64_t M, int64_t K, int64_t ldx, const float *amax, void *q,
                              float *scale, void *stream) {
  int rc = check_rows("quantize_given_amax", x, M, K, ldx);
  if (rc) return rc;
  if (M == 0) return CIDER_OK;
  if (!amax || !q || !scale) return fail(CIDER_E_INVALID, "quantize_given_amax: null pointer");
  return launch_quantize_given_amax(static_cast<const __half *>(x), M, K, ldx, amax, static_cast<int8_t *>(q), scale,
                                    static_cast<cudaStream_t>(stream));
}

int cider_quantize_consume_amax(const void *x, int64_t M, int64_t K, int64_t ldx, float *amax, void *q,
                                float *scale, void *stream) {
  int rc = check_rows("quantize_consume_amax", x, M, K, ldx);
  if (rc) return rc;
  if (M == 0) return CIDER_OK;
  if (!amax || !q || !scale) return fail(CIDER_E_INVALID, "quantize_consume_amax: null pointer");
  return launch_quantize_given_amax(static_cast<const __half *>(x), M, K, ldx, amax, static_cast<int8_t *>(q), scale,
                                    static_cast<cudaStream_t>(stream), true);
}

int cider_swiglu_linear_prequantized(const void *a, const float *sa, const void *w, const float *sw,
                                     const void *bias, void *act, float *rowmax, int64_t M, int64_t N,
                                     int64_t K, void *stream) {
  int rc = check_dims("swiglu_linear_prequantized", M, N, K);
  if (rc) return rc;
  if (N % 64 != 0) return fail(CIDER_E_SHAPE, "swiglu_linear_prequantized: N must be a multiple of 64");
  if (M == 0) return CIDER_OK;
  if (!a || !sa || !w || !sw || !act || !rowmax)
    return fail(CIDER_E_INVALID, "swiglu_linear_prequantized: null pointer");
  GemmArgs g;
  g.a = static_cast<const int8_t *>(a);
  g.b = static_cast<const int8_t *>(w);
  g.out = act; g.sa = sa; g.sw = sw; g.sw_is_half = 0;
  g.bias = static_cast<const __half *>(bias);
  g.M = M; g.N = N; g.K = K; g.gs = 0;
  g.epi = Epi::kPerChannel;
  g.rowmax = rowmax;
  if (!gemm_tc_eligible(g))
    return fail(CIDER_E_SHAPE, "swiglu_linear_prequantized: shape or alignment not supported by the tensor-core kernels");
  return launch_gemm_tc(g, static_cast<cudaStream_t>(stream));
}

int cider_int8_matmul_int32(const void *a, const void *b, int32_t *c, int64_t M, int64_t N, int64_t K,
                            void *stream) {
  if (M < 0 || N < 0 || K < 0) return fail(CIDER_E_INVALID, "int8_matmul_int32: negative size");
  if (M == 0 || N == 0) return CIDER_OK;
  if (!c) return fail(CIDER_E_INVALID, "int8_matmul_int32: null output");
  if (K > 0 && (!a || !b)) return fail(CIDER_E_INVALID, "int8_matmul_int32: null input");
  if (M > (int64_t)1 << 30 || N > (int64_t)1 << 30 || K > (int64_t)1 << 30)
    return fail(CIDER_E_INVALID, "int8_matmul_int32: dimension exceeds 2^30");
  if (reinterpret_cast<uintptr_t>(c) & 3u)
    return fail(CIDER_E_ALIGNMENT, "int8_matmul_int32: output must be 4-byte aligned");
  GemmArgs g;
  g.a = static_cast<const int8_t *>(a);
  g.b = static_cast<const int8_t *>(b);
  g.out = c;
  g.M = M; g.N = N; g.K = K;
  g.epi = Epi::kRawInt32;
  return run_gemm(g, static_cast<cudaStream_t>(stream));
}

int cider_linear_prequantized(const void *a, const float *sa, const void *w, const void *sw, int sw_dtype,
                              int gs, const void *bias, void *y, int64_t M, int64_t N, int64_t K,
                              void *stream) {
  int rc = check_dims("linear_prequantized", M, N, K);
  if (rc) return rc;
  if ((rc = check_dtype("linear_prequantized", sw_dtype))) return rc;
  if (gs != 0 && (rc = check_group("linear_prequantized", K, gs))) return rc;
  if (gs == 0 && sw_dtype != CIDER_F32)
    return fail(CIDER_E_INVALID, "linear_prequantized: per-channel scales must be fp32");
  if (M == 0) return CIDER_OK;
  if (!a || !sa || !w || !sw || !y) return fail(CIDER_E_INVALID, "linear_prequantized: null pointer");
  GemmArgs g;
  g.a = static_cast<const int8_t *>(a);
  g.b = static_cast<const int8_t *>(w);
  g.out = y; g.sa = sa; g.sw = sw; g.sw_is_half = sw_dtype == CIDER_F16;
  g.bias = static_cast<const __half *>(bias);
  g.M = M; g.N = N; g.K = K; g.gs = gs;
  g.epi = gs == 0 ? Epi::kPerChannel : Epi::kPerGroup;
  // a handful of rows: weight streaming kernel instead of a 128-row tensor-core tile
  if (g_backend.load() == 0 && smallm_eligible(M, N, K, gs, a, w, sw))
    return launch_smallm(g.a, sa, g.b, sw, g.sw_is_half, gs, g.bias, static_cast<__half *>(y), M, N, K,
                         static_cast<cudaStream_t>(stream));
  return run_gemm(g, static_cast<cudaStream_t>(stream));
}

int cider_perchannel_linear(const void *x, const void *w, const float *sw, const void *bias, void *y,
                            int64_t M, int64_t N, int64_t K, void *ws, size_t ws_bytes, void *stream) {
  int rc = check_dims("perchannel_linear", M, N, K);
  if (rc) return rc;
  if (M == 0) return CIDER_OK;
  if (!x || !w || !sw || !y) return fail(CIDER_E_INVALID, "perchannel_linear: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (M == 1)
    return launch_gemv(static_cast<const __half *>(x), static_cast<const int8_t *>(w), sw, 0, 0,
                       static_cast<const __half *>(bias), static_cast<__half *>(y), N, K, st);
  Workspace wk;
  if ((rc = carve(CIDER_OP_PERCHANNEL, ws, ws_bytes, M, N, K, &wk))) return rc;
  if ((rc = launch_quantize_per_token(static_cast<const __half *>(x), M, K, K, wk.a_q, wk.sa, st))) return rc;
  // few output tiles and a long K: split-K over int32 slabs in the workspace (bit-identical
  // results: the partial sums are integers)
  const SplitKPlan pl = plan_splitk(M, N, K);
  if (pl.splits >= 2 && wk.splitk != nullptr && g_backend.load() != 1 &&
      !smallm_eligible(M, N, K, 0, wk.a_q, w, sw)) {
    GemmArgs g;
    g.a = wk.a_q;
    g.b = static_cast<const int8_t *>(w);
    g.out = y; g.sa = wk.sa; g.sw = sw; g.sw_is_half = 0;
    g.bias = static_cast<const __half *>(bias);
    g.M = M; g.N = N; g.K = K; g.gs = 0;
    g.epi = Epi::kPerChannel;
    const auto a16 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    if (gemm_tc_eligible(g) && a16(y) && a16(sw)) return launch_gemm_tc_splitk(g, pl, wk.splitk, st);
  }
  return cider_linear_prequantized(wk.a_q, wk.sa, w, sw, CIDER_F32, 0, bias, y, M, N, K, stream);
}

int cider_pergroup_linear(const void *x, const void *w, const void *sw, int sw_dtype, const void *bias,
                          void *y, int64_t M, int64_t N, int64_t K, int gs, void *ws, size_t ws_bytes,
                          void *stream) {
  int rc = check_dims("pergroup_linear", M, N, K);
  if (rc) return rc;
  if ((rc = check_dtype("pergroup_linear", sw_dtype))) return rc;
  if ((rc = check_group("pergroup_linear", K, gs))) return rc;
  if (M == 0) return CIDER_OK;
  if (!x || !w || !sw || !y) return fail(CIDER_E_INVALID, "pergroup_linear: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (M == 1)
    return launch_gemv(static_cast<const __half *>(x), static_cast<const int8_t *>(w), sw,
                       sw_dtype == CIDER_F16, gs, static_cast<const __half *>(bias),
                       static_cast<__half *>(y), N, K, st);
  Workspace wk;
  if ((rc = carve(CIDER_OP_PERGROUP, ws, ws_bytes, M, N, K, &wk))) return rc;
  if ((rc = launch_quantize_per_token(static_cast<const __half *>(x), M, K, K, wk.a_q, wk.sa, st))) return rc;
  // few output tiles and a long K: equal K pieces of whole groups over fp32 slabs in the workspace
  const SplitKPlan pl = plan_pg_splitk(M, N, K);
  if (pl.splits >= 2 && wk.splitk != nullptr && g_backend.load() != 1 &&
      !smallm_eligible(M, N, K, gs, wk.a_q, w, sw)) {
    GemmArgs g;
    g.a = wk.a_q;
    g.b = static_cast<const int8_t *>(w);
    g.out = y; g.sa = wk.sa; g.sw = sw; g.sw_is_half = sw_dtype == CIDER_F16;
    g.bias = static_cast<const __half *>(bias);
    g.M = M; g.N = N; g.K = K; g.gs = gs;
    g.epi = Epi::kPerGroup;
    if (gemm_tc_eligible(g) && (reinterpret_cast<uintptr_t>(y) & 7u) == 0)
      return launch_gemm_tc_pg_splitk(g, pl, wk.splitk, st);
  }
  return cider_linear_prequantized(wk.a_q, wk.sa, w, sw, sw_dtype, gs, bias, y, M, N, K, stream);
}

// W4A8 on packed rows [N, K/2] with quantised activations at hand: the streaming kernel
// for a handful of rows, else the tensor-core kernels, both of which expand the nibbles
// themselves (no int8 copy of the weights exists anywhere).
// Quantise x for w4_rows_linear.  The tensor-core kernels expand the nibbles of 8 k in the order
// k0 k2 k4 k6 k1 k3 k5 k7 and want the activations in the same order; the streaming kernel for a
// handful of rows takes them in natural order.
static bool w4_rows_streams(const Workspace &wk, const uint8_t *w_rows, const void *sw, int gs, int64_t M, int64_t N,
                            int64_t K) {
  return g_backend.load() == 0 && smallm_eligible(M, N, K, gs, wk.a_q, w_rows, sw, true);
}
static int w4_rows_quantize(const Workspace &wk, const void *x, const uint8_t *w_rows, const void *sw, int gs,
                            int64_t M, int64_t N, int64_t K, cudaStream_t st) {
  const __half *xh = static_cast<const __half *>(x);
  if (w4_rows_streams(wk, w_rows, sw, gs, M, N, K)) return launch_quantize_per_token(xh, M, K, K, wk.a_q, wk.sa, st);
  if (quantize_perm8_ok(xh, K, K, wk.a_q)) return launch_quantize_per_token_perm8(xh, M, K, K, wk.a_q, wk.sa, st);
  int rc = launch_quantize_per_token(xh, M, K, K, wk.a_q, wk.sa, st);
  if (rc) return rc;
  return launch_permute8(wk.a_q, M * K, st);  // K % 32 == 0 on this path
}

// (activations from w4_rows_quantize)
static int w4_rows_linear(const Workspace &wk, const uint8_t *w_rows, const void *sw, int sw_dtype, int gs, void *y,
                          int64_t M, int64_t N, int64_t K, cudaStream_t st) {
  const bool sw_half = sw_dtype == CIDER_F16;
  const int backend = g_backend.load();
  if (w4_rows_streams(wk, w_rows, sw, gs, M, N, K))
    return launch_smallm(wk.a_q, wk.sa, reinterpret_cast<const int8_t *>(w_rows), sw, sw_half, gs, nullptr,
                         static_cast<__half *>(y), M, N, K, st, true);
  GemmArgs g;
  g.a = wk.a_q;
  g.w4rows = w_rows;
  g.out = y; g.sa = wk.sa; g.sw = sw; g.sw_is_half = sw_half;
  g.M = M; g.N = N; g.K = K; g.gs = gs;
  g.epi = gs == 0 ? Epi::kPerChannel : Epi::kPerGroup;
  if (backend != 1 && gemm_tc_eligible(g)) return launch_gemm_tc(g, st);
  return fail(CIDER_E_SHAPE, "w4a8: the packed-row kernels do not take this shape / alignment / backend");
}

int cider_w4a8_linear(const void *x, const void *packed_w, const void *sw, int sw_dtype, int gs, void *y,
                      int64_t M, int64_t N, int64_t K, void *ws, size_t ws_bytes, void *stream) {
  int rc = check_dims("w4a8_linear", M, N, K);
  if (rc) return rc;
  if ((rc = check_dtype("w4a8_linear", sw_dtype))) return rc;
  if (K % 2 != 0) return fail(CIDER_E_SHAPE, "w4a8_linear: K must be even");
  if (gs != 0 && (rc = check_group("w4a8_linear", K, gs))) return rc;
  if (M == 0) return CIDER_OK;
  if (!x || !packed_w || !sw || !y) return fail(CIDER_E_INVALID, "w4a8_linear: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Workspace wk;
  if ((rc = carve(CIDER_OP_W4A8, ws, ws_bytes, M, N, K, &wk))) return rc;
  const int backend = g_backend.load();
  // The reference's [K/2, N] packing (N contiguous) cannot be read row by row: one byte
  // transpose into rows ([N, K/2], half the bytes of an int8 copy) in the workspace, then
  // the packed-row kernels.
  if (backend != 1 && wk.w_scratch != nullptr) {
    if ((rc = w4_rows_quantize(wk, x, wk.w_scratch, sw, gs, M, N, K, st))) return rc;
    if ((rc = launch_repack_w4(static_cast<const uint8_t *>(packed_w), wk.w_scratch, N, K, st))) return rc;
    return w4_rows_linear(wk, wk.w_scratch, sw, sw_dtype, gs, y, M, N, K, st);
  }
  if ((rc = launch_quantize_per_token(static_cast<const __half *>(x), M, K, K, wk.a_q, wk.sa, st))) return rc;
  if (backend == 2)
    return fail(CIDER_E_SHAPE, "tensor-core GEMM requested but the shape / alignment does not allow it");
  // other shapes (K < 128, K % 32 != 0) and the plain backend: the CUDA-core kernel reads
  // the packed bytes in place
  GemmArgs g;
  g.a = wk.a_q;
  g.out = y; g.sa = wk.sa; g.sw = sw; g.sw_is_half = sw_dtype == CIDER_F16;
  g.M = M; g.N = N; g.K = K; g.gs = gs;
  g.epi = gs == 0 ? Epi::kPerChannel : Epi::kPerGroup;
  g.packed4 = static_cast<const uint8_t *>(packed_w);
  return launch_gemm_generic(g, st);
}

int cider_w4a8_repack(const void *packed_w, void *w_nk4, int64_t N, int64_t K, void *stream) {
  if (N < 0 || K < 0 || (K % 2) != 0) return fail(CIDER_E_SHAPE, "w4a8_repack: K must be even, N and K >= 0");
  if (N == 0 || K == 0) return CIDER_OK;
  if (!packed_w || !w_nk4) return fail(CIDER_E_INVALID, "w4a8_repack: null pointer");
  return launch_repack_w4(static_cast<const uint8_t *>(packed_w), static_cast<uint8_t *>(w_nk4), N, K,
                          static_cast<cudaStream_t>(stream));
}

int cider_w4a8_linear_nk4(const void *x, const void *w_nk4, const void *sw, int sw_dtype, int gs, void *y,
                          int64_t M, int64_t N, int64_t K, void *ws, size_t ws_bytes, void *stream) {
  int rc = check_dims("w4a8_linear_nk4", M, N, K);
  if (rc) return rc;
  if ((rc = check_dtype("w4a8_linear_nk4", sw_dtype))) return rc;
  if (K % 16 != 0) return fail(CIDER_E_SHAPE, "w4a8_linear_nk4: K must be a multiple of 16");
  if (gs != 0 && (rc = check_group("w4a8_linear_nk4", K, gs))) return rc;
  if (M == 0) return CIDER_OK;
  if (!x || !w_nk4 || !sw || !y) return fail(CIDER_E_INVALID, "w4a8_linear_nk4: null pointer");
  if (reinterpret_cast<uintptr_t>(w_nk4) & 15u)
    return fail(CIDER_E_INVALID, "w4a8_linear_nk4: weights must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Workspace wk;
  // A caller that lends N*K more bytes than the packed-row kernels need (CIDER_OP_W4A8_ROWS_INT8COPY)
  // trades memory for time: beyond decode sizes the weights are then expanded to an int8 copy by
  // a pass of their own and the int8 kernels run on it.
  // (from the sizes on where the copy pays: measured on [10240, 2560], the expanding pass costs
  // ~8 us and the in-kernel expansion 14 % per channel / 30 % per group of the GEMM time)
  const bool int8copy = w4_rows_shape(K) && ws != nullptr && M >= (gs ? 256 : 2048) &&
                        ws_bytes >= workspace_bytes(CIDER_OP_W4A8_ROWS_INT8COPY, M, N, K) &&
                        g_backend.load() != 1;
  const int op = int8copy ? CIDER_OP_W4A8_ROWS_INT8COPY : CIDER_OP_W4A8_ROWS;
  if ((rc = carve(op, ws, ws_bytes, M, N, K, &wk))) return rc;
  if (wk.w_scratch == nullptr) {  // K >= 128, K % 32 == 0: the kernels read the packed rows
    if ((rc = w4_rows_quantize(wk, x, static_cast<const uint8_t *>(w_nk4), sw, gs, M, N, K, st))) return rc;
    return w4_rows_linear(wk, static_cast<const uint8_t *>(w_nk4), sw, sw_dtype, gs, y, M, N, K, st);
  }
  if ((rc = launch_quantize_per_token(static_cast<const __half *>(x), M, K, K, wk.a_q, wk.sa, st))) return rc;
  // odd shapes, or scratch lent for it: an int8 copy in the workspace, then the int8 kernels
  const bool sw_half = sw_dtype == CIDER_F16;
  if (g_backend.load() == 0 && smallm_eligible(M, N, K, gs, wk.a_q, w_nk4, sw, true))
    return launch_smallm(wk.a_q, wk.sa, static_cast<const int8_t *>(w_nk4), sw, sw_half, gs, nullptr,
                         static_cast<__half *>(y), M, N, K, st, true);
  int8_t *w8 = reinterpret_cast<int8_t *>(wk.w_scratch);
  if ((rc = launch_unpack_w4_nk(static_cast<const uint8_t *>(w_nk4), w8, N, K, st))) return rc;
  return cider_linear_prequantized(wk.a_q, wk.sa, w8, sw, sw_dtype, gs, nullptr, y, M, N, K, stream);
}

int cider_rmsnorm_quant(const void *x, const void *w, float eps, int64_t M, int64_t K, void *y, void *q,
                        float *scale, void *stream) {
  if (M < 0 || K <= 0) return fail(CIDER_E_INVALID, "rmsnorm_quant: need M >= 0, K > 0");
  if (M == 0) return CIDER_OK;
  if (!x || !w || !q || !scale) return fail(CIDER_E_INVALID, "rmsnorm_quant: null pointer");
  if (M > (int64_t)1 << 30 || K > (int64_t)1 << 30)
    return fail(CIDER_E_INVALID, "rmsnorm_quant: dimension exceeds 2^30");
  return launch_rmsnorm_quant(static_cast<const __half *>(x), static_cast<const __half *>(w), eps, M, K,
                              static_cast<__half *>(y), static_cast<int8_t *>(q), scale,
                              static_cast<cudaStream_t>(stream));
}

int cider_add_rmsnorm_quant(void *x, const void *delta, const void *w, float eps, int64_t M, int64_t K,
                            void *y, void *q, float *scale, void *stream) {
  if (M < 0 || K <= 0) return fail(CIDER_E_INVALID, "add_rmsnorm_quant: need M >= 0, K > 0");
  if (M == 0) return CIDER_OK;
  if (!x || !w) return fail(CIDER_E_INVALID, "add_rmsnorm_quant: null pointer");
  if (!y && !q) return fail(CIDER_E_INVALID, "add_rmsnorm_quant: neither an fp16 nor an int8 output given");
  if (q && !scale) return fail(CIDER_E_INVALID, "add_rmsnorm_quant: int8 output without a scale output");
  if (M > (int64_t)1 << 30 || K > (int64_t)1 << 30)
    return fail(CIDER_E_INVALID, "add_rmsnorm_quant: dimension exceeds 2^30");
  return launch_add_rmsnorm_quant(static_cast<__half *>(x), static_cast<const __half *>(delta),
                                  static_cast<const __half *>(w), eps, M, K, static_cast<__half *>(y),
                                  static_cast<int8_t *>(q), scale, static_cast<cudaStream_t>(stream));
}

int cider_qk_norm_rope_append(const void *qkv, const void *q_norm_w, const void *k_norm_w,
                              const float *inv_freq, const int8_t *axis, const int32_t *pos3,
                              int64_t pos_stride, const int32_t *base_dev, int64_t base_host, float eps,
                              void *q_out, void *k_cache, void *v_cache, int64_t B, int64_t T, int64_t nq,
                              int64_t nkv, int64_t D, int64_t Tcap, void *stream) {
  if (B < 0 || T < 0 || nq <= 0 || nkv <= 0 || Tcap <= 0 || base_host < 0)
    return fail(CIDER_E_INVALID, "qk_norm_rope_append: bad sizes");
  if (D != 128) return fail(CIDER_E_SHAPE, "qk_norm_rope_append: head_dim must be 128");
  if (B * T == 0) return CIDER_OK;
  if (!qkv || !q_norm_w || !k_norm_w || !inv_freq || !axis || !pos3 || !q_out || !k_cache || !v_cache)
    return fail(CIDER_E_INVALID, "qk_norm_rope_append: null pointer");
  if (!base_dev && base_host + T > Tcap) return fail(CIDER_E_SHAPE, "qk_norm_rope_append: cache overflow");
  if (B * T > 0x7fffffff || nq + 2 * nkv > 65535) return fail(CIDER_E_SHAPE, "qk_norm_rope_append: too large");
  for (const void *ptr : {qkv, q_norm_w, k_norm_w, (const void *)q_out, (const void *)k_cache, (const void *)v_cache})
    if (reinterpret_cast<uintptr_t>(ptr) & 15u)
      return fail(CIDER_E_ALIGNMENT, "qk_norm_rope_append: fp16 buffers must be 16-byte aligned");
  return launch_qk_norm_rope_append(static_cast<const __half *>(qkv), static_cast<const __half *>(q_norm_w),
                                    static_cast<const __half *>(k_norm_w), inv_freq, axis, pos3,
                                    (int)pos_stride, base_dev, (int)base_host, eps,
                                    static_cast<__half *>(q_out), static_cast<__half *>(k_cache),
                                    static_cast<__half *>(v_cache), B, T, (int)nq, (int)nkv, Tcap,
                                    static_cast<cudaStream_t>(stream));
}

int cider_silu_mul(const void *gate_up, void *act, int64_t M, int64_t inter, void *stream) {
  if (M < 0 || inter <= 0 || inter % 2) return fail(CIDER_E_INVALID, "silu_mul: need M >= 0 and an even inter > 0");
  if (M == 0) return CIDER_OK;
  if (!gate_up || !act) return fail(CIDER_E_INVALID, "silu_mul: null pointer");
  return launch_silu_mul(static_cast<const __half *>(gate_up), static_cast<__half *>(act), M, inter,
                         static_cast<cudaStream_t>(stream));
}

int cider_quantize_heads(const void *a, int64_t B, int64_t heads, int64_t T, int64_t D, void *q, float *scale,
                         void *stream) {
  if (B < 0 || heads <= 0 || T < 0 || D <= 0) return fail(CIDER_E_INVALID, "quantize_heads: bad sizes");
  if (B * T == 0) return CIDER_OK;
  if (!a || !q || !scale) return fail(CIDER_E_INVALID, "quantize_heads: null pointer");
  if (B * T > 0x7fffffff || heads * D > 0x7fffffff) return fail(CIDER_E_SHAPE, "quantize_heads: too large");
  return launch_quantize_heads(static_cast<const __half *>(a), B, heads, T, D, static_cast<int8_t *>(q), scale,
                               static_cast<cudaStream_t>(stream));
}

int cider_silu_mul_quant(const void *gate_up, int64_t M, int64_t inter, void *q, float *scale, void *stream) {
  if (M < 0 || inter < 0) return fail(CIDER_E_INVALID, "silu_mul_quant: negative dimension");
  if (M == 0) return CIDER_OK;
  if (!gate_up || !q || !scale) return fail(CIDER_E_INVALID, "silu_mul_quant: null pointer");
  return launch_silu_mul_quant(static_cast<const __half *>(gate_up), M, inter, static_cast<int8_t *>(q), scale,
                               static_cast<cudaStream_t>(stream));
}

int cider_linear_m1_fused(const void *x, int prologue, const void *delta, const void *norm_w, float eps,
                          void *x_out, const void *w, const void *sw, int sw_dtype, int gs, const void *bias,
                          void *y, int64_t N, int64_t K, void *stream) {
  int rc = check_dims("linear_m1_fused", 1, N, K);
  if (rc) return rc;
  if ((rc = check_dtype("linear_m1_fused", sw_dtype))) return rc;
  if (gs != 0 && (rc = check_group("linear_m1_fused", K, gs))) return rc;
  if (gs == 0 && sw_dtype != CIDER_F32) return fail(CIDER_E_INVALID, "linear_m1_fused: per-channel scales must be fp32");
  if (prologue < 0 || prologue > 2) return fail(CIDER_E_INVALID, "linear_m1_fused: prologue must be 0, 1 or 2");
  if (!x || !w || !sw || !y) return fail(CIDER_E_INVALID, "linear_m1_fused: null pointer");
  if (prologue == 2 && !norm_w) return fail(CIDER_E_INVALID, "linear_m1_fused: add+norm prologue needs a norm weight");
  if (prologue == 2 && x_out == x) return fail(CIDER_E_INVALID, "linear_m1_fused: x_out must not alias x");
  auto a16 = [](const void *p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!a16(x) || !a16(delta) || !a16(norm_w) || !a16(x_out))
    return fail(CIDER_E_ALIGNMENT, "linear_m1_fused: activation pointers must be 16-byte aligned");
  return launch_gemv_fused(static_cast<const __half *>(x), prologue, static_cast<const __half *>(delta),
                           static_cast<const __half *>(norm_w), eps, static_cast<__half *>(x_out),
                           static_cast<const int8_t *>(w), sw, sw_dtype == CIDER_F16, gs,
                           static_cast<const __half *>(bias), static_cast<__half *>(y), N, K,
                           static_cast<cudaStream_t>(stream));
}

size_t cider_sdpa_decode_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t D, int64_t T) {
  return sdpa_decode_workspace_bytes(B, Hq, Hkv, D, T);
}

static int sdpa_decode_impl(const void *q, const void *kc, const void *vc, void *out, int64_t B, int64_t Hq,
                            int64_t Hkv, int64_t D, int64_t T, int64_t Tcap, float scale, void *ws,
                            size_t ws_bytes, const int32_t *length_dev, uint32_t *tickets, void *stream) {
  if (B < 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || T < 0 || Tcap < T)
    return fail(CIDER_E_INVALID, "sdpa_decode: bad sizes");
  if (Hq % Hkv != 0) return fail(CIDER_E_SHAPE, "sdpa_decode: Hq must be a multiple of Hkv");
  if (D != 64 && D != 128) return fail(CIDER_E_SHAPE, "sdpa_decode: head_dim must be 64 or 128");
  if (B == 0) return CIDER_OK;
  if (!q || !out || (T > 0 && (!kc || !vc))) return fail(CIDER_E_INVALID, "sdpa_decode: null pointer");
  return launch_sdpa_decode(static_cast<const __half *>(q), static_cast<const __half *>(kc),
                            static_cast<const __half *>(vc), static_cast<__half *>(out), B, Hq, Hkv, D, T,
                            Tcap, scale, ws, ws_bytes, length_dev, tickets, static_cast<cudaStream_t>(stream));
}

int cider_sdpa_decode(const void *q, const void *kc, const void *vc, void *out, int64_t B, int64_t Hq,
                      int64_t Hkv, int64_t D, int64_t T, int64_t Tcap, float scale, void *ws,
                      size_t ws_bytes, const int32_t *length_dev, void *stream) {
  return sdpa_decode_impl(q, kc, vc, out, B, Hq, Hkv, D, T, Tcap, scale, ws, ws_bytes, length_dev, nullptr, stream);
}

int cider_sdpa_decode_tickets(const void *q, const void *kc, const void *vc, void *out, int64_t B, int64_t Hq,
                              int64_t Hkv, int64_t D, int64_t T, int64_t Tcap, float scale, void *ws,
                              size_t ws_bytes, const int32_t *length_dev, uint32_t *tickets, void *stream) {
  if (B > 0 && !tickets) return fail(CIDER_E_INVALID, "sdpa_decode_tickets: null ticket buffer");
  return sdpa_decode_impl(q, kc, vc, out, B, Hq, Hkv, D, T, Tcap, scale, ws, ws_bytes, length_dev, tickets, stream);
}

int cider_sdpa_decode_fused(const void *qkv, const void *q_norm_w, const void *k_norm_w, const float *inv_freq,
                            const int8_t *axis, const int32_t *pos3, int64_t pos_stride, float eps, void *kc, void *vc,
                            void *out, int64_t B, int64_t Hq, int64_t Hkv, int64_t D, int64_t T, int64_t Tcap,
                            float scale, void *ws, size_t ws_bytes, const int32_t *length_dev, uint32_t *tickets,
                            void *stream) {
  if (B < 0 || Hq <= 0 || Hkv <= 0 || T < 1 || Tcap < T) return fail(CIDER_E_INVALID, "sdpa_decode_fused: bad sizes");
  if (Hq % Hkv != 0) return fail(CIDER_E_SHAPE, "sdpa_decode_fused: Hq must be a multiple of Hkv");
  if (D != 128) return fail(CIDER_E_SHAPE, "sdpa_decode_fused: head_dim must be 128");
  if (B == 0) return CIDER_OK;
  if (!qkv || !q_norm_w || !k_norm_w || !inv_freq || !axis || !pos3 || !kc || !vc || !out)
    return fail(CIDER_E_INVALID, "sdpa_decode_fused: null pointer");
  for (const void *ptr : {qkv, q_norm_w, k_norm_w})
    if (reinterpret_cast<uintptr_t>(ptr) & 15u)
      return fail(CIDER_E_ALIGNMENT, "sdpa_decode_fused: fp16 buffers must be 16-byte aligned");
  return launch_sdpa_decode_fused(static_cast<const __half *>(qkv), static_cast<const __half *>(q_norm_w),
                                  static_cast<const __half *>(k_norm_w), inv_freq, axis, pos3, (int)pos_stride, eps,
                                  static_cast<__half *>(kc), static_cast<__half *>(vc), static_cast<__half *>(out), B,
                                  Hq, Hkv, T, Tcap, scale, ws, ws_bytes, length_dev, tickets,
                                  static_cast<cudaStream_t>(stream));
}

int cider_device_status(unsigned int *status) {
  if (!status) return fail(CIDER_E_INVALID, "device_status: null pointer");
  return read_device_status(status);
}

int cider_clear_device_status(void) { return clear_device_status(); }

int cider_set_programmatic_launch(int enable) {
  g_pdl.store(enable ? 1 : 0);
  return CIDER_OK;
}

int cider_set_gemm_backend(int backend) {
  if (backend < 0 || backend > 2) return fail(CIDER_E_INVALID, "set_gemm_backend: 0, 1 or 2");
  g_backend.store(backend);
  return CIDER_OK;
}

int cider_testing_set_tile(int tile, int bn) { return set_tile_override(tile, bn); }

const char *cider_testing_last_gemm_kernel(void) { return last_gemm_kernel(); }

int cider_testing_set_sdpa_kernel(int mode) { return set_sdpa_kernel(mode); }

}  // extern "C"
