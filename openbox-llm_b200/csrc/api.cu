// C-ABI entry points of the attention branches: argument checks, kernel-family choice,
// workspace carving.  The kernels live in simt.cu (CUDA cores) and tc.cu (tcgen05 / TMEM).
#include <stdarg.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"

namespace nsa {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

// One status word per device, raised (atomicOr) by kernels whose bounded waits run out.
__device__ int g_device_status = 0;

int* device_status_ptr() {
  int* p = nullptr;
  if (cudaGetSymbolAddress((void**)&p, g_device_status) != cudaSuccess) return nullptr;
  return p;
}

// ---- kernel accounting ---------------------------------------------------------------------
static std::atomic<long long> g_launches{0};
static std::atomic<int> g_profile{0};
struct ProfRec { std::string name; cudaEvent_t e0, e1; };
static std::mutex g_prof_mu;
static std::vector<ProfRec> g_prof;
static thread_local cudaEvent_t t_open_e1 = nullptr;

void kernel_begin(const char* name, cudaStream_t st) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  t_open_e1 = nullptr;
  if (!g_profile.load(std::memory_order_relaxed)) return;
  ProfRec r;
  r.name = name;
  if (cudaEventCreate(&r.e0) != cudaSuccess || cudaEventCreate(&r.e1) != cudaSuccess) return;
  cudaEventRecord(r.e0, st);
  t_open_e1 = r.e1;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  g_prof.push_back(r);
}

void kernel_end(cudaStream_t st) {
  if (t_open_e1) cudaEventRecord(t_open_e1, st);
  t_open_e1 = nullptr;
}

static std::atomic<int> g_opt_sel_fwd{0};
int get_option_sel_fwd() { return g_opt_sel_fwd.load(); }
static std::atomic<int> g_opt_bwd_kernel{1};
int get_option_bwd_kernel() { return g_opt_bwd_kernel.load(); }
static std::atomic<int> g_opt_merged{1};
int get_option_merged_boxes() { return g_opt_merged.load(); }
static std::atomic<int> g_opt_starve{0};
int get_option_debug_starve_load() { return g_opt_starve.load(); }

static int check_dims(const NsaDims* d) {
  NSA_CHECK_ARG(d != nullptr, "dims is null");
  NSA_CHECK_ARG(d->B >= 0 && d->T >= 0 && d->Hq > 0 && d->Hkv > 0, "bad B/T/Hq/Hkv");
  NSA_CHECK_ARG(d->Hq % d->Hkv == 0, "Hq=%d is not a multiple of Hkv=%d", d->Hq, d->Hkv);
  NSA_CHECK_ARG(d->D == 16 || d->D == 32 || d->D == 64 || d->D == 128,
                "head dim must be a power of two <= 128, got %d", d->D);   // nsa_selection_kernel.py:187
  NSA_CHECK_ARG(d->dtype == NSA_DTYPE_BF16 || d->dtype == NSA_DTYPE_F32, "bad dtype %d", d->dtype);
  return NSA_OK;
}

static size_t elem_size(int dtype) { return dtype == NSA_DTYPE_BF16 ? 2 : 4; }

static AttnArgs base_args(const NsaDims* d, int Lk) {
  AttnArgs a;
  memset(&a, 0, sizeof(a));
  a.B = d->B; a.Hq = d->Hq; a.Hkv = d->Hkv; a.T = d->T; a.D = d->D; a.Lk = Lk;
  a.scale = 1.0f / sqrtf((float)d->D);
  return a;
}

static bool use_tc(const NsaDims* d, int block_size, int impl, int* err) {
  *err = NSA_OK;
  if (impl == NSA_IMPL_SIMT) return false;
  const bool ok = tc_shape_ok(*d, block_size);
  if (impl == NSA_IMPL_TC && !ok) {
    set_error("shape not served by the tcgen05 kernels (bf16, D in {64,128}, 64-token blocks, 2 to 128 query heads per kv head)");
    *err = NSA_ERR_UNSUPPORTED;
  }
  return ok;
}

// backward through the SIMT kernels: dq direct, dk/dv via fp32 accumulators
static size_t simt_bwd_ws(const NsaDims* d, int Lk) {
  if (d->dtype == NSA_DTYPE_F32) return 0;   // accumulate straight into dk/dv
  return 2 * align_up((size_t)d->B * d->Hkv * Lk * d->D * sizeof(float), 256);
}

static int simt_bwd(AttnArgs& a, const NsaDims* d, void* dk, void* dv, void* ws, size_t ws_bytes,
                    cudaStream_t st) {
  const size_t n = (size_t)d->B * d->Hkv * a.Lk * d->D;
  if (d->dtype == NSA_DTYPE_F32) {
    a.dk_acc = (float*)dk;
    a.dv_acc = (float*)dv;
  } else {
    if (ws_bytes < simt_bwd_ws(d, a.Lk) || (!ws && n)) {
      set_error("backward workspace too small: need %zu bytes", simt_bwd_ws(d, a.Lk));
      return NSA_ERR_WORKSPACE;
    }
    a.dk_acc = (float*)ws;
    a.dv_acc = (float*)((char*)ws + align_up(n * sizeof(float), 256));
  }
  if (n) {
    NSA_CUDA_OK(cudaMemsetAsync(a.dk_acc, 0, n * sizeof(float), st));
    NSA_CUDA_OK(cudaMemsetAsync(a.dv_acc, 0, n * sizeof(float), st));
  }
  int rc = simt_attn_bwd(a, d->dtype, st);
  if (rc != NSA_OK) return rc;
  if (d->dtype != NSA_DTYPE_F32) {
    rc = cast_f32_to(a.dk_acc, dk, n, d->dtype, st);
    if (rc != NSA_OK) return rc;
    rc = cast_f32_to(a.dv_acc, dv, n, d->dtype, st);
  }
  return rc;
}

}  // namespace nsa

using namespace nsa;

extern "C" const char* nsa_last_error(void) { return g_err; }
extern "C" int nsa_version(void) { return 100; }

extern "C" int nsa_tc_supported(const NsaDims* dims, int block_size) {
  if (check_dims(dims) != NSA_OK) return 0;
  return tc_shape_ok(*dims, block_size) ? 1 : 0;
}

extern "C" long long nsa_launch_count(void) { return g_launches.load(); }

extern "C" int nsa_set_option(const char* name, int value) {
  if (name && strcmp(name, "sel_fwd_variant") == 0 && value >= 0 && value <= 2) {
    g_opt_sel_fwd.store(value);
    return NSA_OK;
  }
  if (name && strcmp(name, "bwd_kernel") == 0 && value >= 0 && value <= 1) {
    g_opt_bwd_kernel.store(value);
    return NSA_OK;
  }
  if (name && strcmp(name, "merged_boxes") == 0 && value >= 0 && value <= 1) {
    g_opt_merged.store(value);
    return NSA_OK;
  }
  if (name && strcmp(name, "debug_starve_load") == 0 && value >= 0 && value <= 1) {
    g_opt_starve.store(value);
    return NSA_OK;
  }
  set_error("unknown option or value");
  return NSA_ERR_BAD_ARG;
}

extern "C" void nsa_profile_enable(int on) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  for (auto& r : g_prof) { cudaEventDestroy(r.e0); cudaEventDestroy(r.e1); }
  g_prof.clear();
  g_profile.store(on ? 1 : 0);
}

extern "C" int nsa_profile_summary(char* buf, size_t cap) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  std::vector<std::string> names;
  std::vector<double> ms;
  std::vector<long long> cnt;
  for (auto& r : g_prof) {
    if (cudaEventSynchronize(r.e1) != cudaSuccess) continue;
    float t = 0.f;
    if (cudaEventElapsedTime(&t, r.e0, r.e1) != cudaSuccess) continue;
    size_t i = 0;
    for (; i < names.size(); ++i) if (names[i] == r.name) break;
    if (i == names.size()) { names.push_back(r.name); ms.push_back(0); cnt.push_back(0); }
    ms[i] += t; cnt[i] += 1;
  }
  size_t off = 0;
  if (cap) buf[0] = 0;
  for (size_t i = 0; i < names.size(); ++i) {
    int n = snprintf(buf + off, off < cap ? cap - off : 0, "%s %lld %.6f\n", names[i].c_str(), cnt[i], ms[i]);
    if (n < 0 || off + (size_t)n >= cap) break;
    off += (size_t)n;
  }
  return (int)names.size();
}

extern "C" int nsa_device_status(void* stream) {
  int* p = device_status_ptr();
  if (!p) { set_error("cudaGetSymbolAddress failed"); return NSA_ERR_CUDA; }
  int v = 0;
  NSA_CUDA_OK(cudaMemcpyAsync(&v, p, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  NSA_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
  if (v != 0) {
    set_error("a kernel gave up a bounded wait (status word 0x%x)", v);
    int zero = 0;
    cudaMemcpyAsync(p, &zero, sizeof(int), cudaMemcpyHostToDevice, (cudaStream_t)stream);
    cudaStreamSynchronize((cudaStream_t)stream);
    return NSA_ERR_DEVICE_WAIT;
  }
  return NSA_OK;
}

extern "C" int nsa_debug_set_device_status(int value, void* stream) {
  int* p = device_status_ptr();
  if (!p) { set_error("cudaGetSymbolAddress failed"); return NSA_ERR_CUDA; }
  // the value travels inside the call (pageable 4-byte source: copied before the call returns)
  NSA_CUDA_OK(cudaMemcpyAsync(p, &value, sizeof(int), cudaMemcpyHostToDevice, (cudaStream_t)stream));
  NSA_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
  return NSA_OK;
}

// ---- range attention -------------------------------------------------------------------------
extern "C" int nsa_range_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                                  const NsaDims* dims, int Lk, int mode, int window, int block_size,
                                  int impl, void* stream) {
  int rc = check_dims(dims);
  if (rc != NSA_OK) return rc;
  NSA_CHECK_ARG(mode == NSA_MODE_WINDOW || mode == NSA_MODE_COMPRESS || mode == NSA_MODE_COMPRESS_STRIDED,
                "bad mode %d", mode);
  NSA_CHECK_ARG(Lk >= 0, "bad Lk");
  if (mode == NSA_MODE_WINDOW) NSA_CHECK_ARG(window >= 1, "window must be >= 1");
  if (mode != NSA_MODE_WINDOW) NSA_CHECK_ARG(block_size >= 1, "block_size must be >= 1");
  const size_t rows = (size_t)dims->B * dims->Hq * dims->T;
  if (rows == 0) return NSA_OK;
  NSA_CHECK_ARG(q && o && lse && (Lk == 0 || (k && v)), "null tensor");
  AttnArgs a = base_args(dims, Lk);
  a.q = q; a.k = k; a.v = v; a.o = o; a.lse = lse;
  a.kind = mode; a.window = window; a.block_size = block_size;
  if (mode == NSA_MODE_COMPRESS) a.window = block_size;   // internally `window` holds the summary stride
  if (mode == NSA_MODE_COMPRESS_STRIDED) {
    NSA_CHECK_ARG(window >= 1 && window <= block_size, "summary stride must be in [1, block_size]");
    a.kind = NSA_MODE_COMPRESS;
  }
  if (use_tc(dims, 64, impl, &rc) && Lk > 0) return tc_attn_fwd(a, (cudaStream_t)stream);
  if (rc != NSA_OK) return rc;
  return simt_attn_fwd(a, dims->dtype, (cudaStream_t)stream);
}

static size_t range_bwd_ws(const NsaDims* dims, int Lk, int mode, int window, int impl, bool acc) {
  if (check_dims(dims) != NSA_OK) return 0;
  int rc;
  size_t need = acc ? 0 : simt_bwd_ws(dims, Lk);
  if (use_tc(dims, 64, impl, &rc)) {
    AttnArgs a = base_args(dims, Lk);
    a.kind = mode == NSA_MODE_COMPRESS_STRIDED ? NSA_MODE_COMPRESS : mode;
    a.window = window > 0 ? window : 1;
    if (acc) a.dq_acc = reinterpret_cast<float*>(sizeof(float));   // only "not null" matters for the plan
    need = need > tc_attn_bwd_workspace(a) ? need : tc_attn_bwd_workspace(a);
  }
  return need;
}

extern "C" size_t nsa_range_attn_bwd_workspace_bytes(const NsaDims* dims, int Lk, int mode,
                                                     int window, int impl) {
  return range_bwd_ws(dims, Lk, mode, window, impl, false);
}

extern "C" size_t nsa_range_attn_bwd_acc_workspace_bytes(const NsaDims* dims, int Lk, int mode,
                                                         int window) {
  return range_bwd_ws(dims, Lk, mode, window, NSA_IMPL_TC, true);
}

static int range_attn_bwd(const void* q, const void* k, const void* v, const void* o,
                          const float* lse, const void* d_o, void* dq, float* dq_acc, void* dk, void* dv,
                          const NsaDims* dims, int Lk, int mode, int window, int block_size,
                          const float* row_scale, const float* row_dot,
                          void* workspace, size_t workspace_bytes, int impl, void* stream) {
  int rc = check_dims(dims);
  if (rc != NSA_OK) return rc;
  NSA_CHECK_ARG(mode == NSA_MODE_WINDOW || mode == NSA_MODE_COMPRESS || mode == NSA_MODE_COMPRESS_STRIDED,
                "bad mode %d", mode);
  if (mode == NSA_MODE_WINDOW) NSA_CHECK_ARG(window >= 1, "window must be >= 1");
  if (mode != NSA_MODE_WINDOW) NSA_CHECK_ARG(block_size >= 1, "block_size must be >= 1");
  cudaStream_t st = (cudaStream_t)stream;
  const size_t rows = (size_t)dims->B * dims->Hq * dims->T;
  const size_t nkv = (size_t)dims->B * dims->Hkv * Lk * dims->D;
  if (rows == 0 || Lk == 0) {
    if (rows && dq) NSA_CUDA_OK(cudaMemsetAsync(dq, 0, rows * dims->D * elem_size(dims->dtype), st));
    if (nkv) {
      NSA_CUDA_OK(cudaMemsetAsync(dk, 0, nkv * elem_size(dims->dtype), st));
      NSA_CUDA_OK(cudaMemsetAsync(dv, 0, nkv * elem_size(dims->dtype), st));
    }
    return NSA_OK;
  }
  NSA_CHECK_ARG(q && k && v && o && lse && d_o && dk && dv, "null tensor");
  AttnArgs a = base_args(dims, Lk);
  a.q = q; a.k = k; a.v = v; a.o = (void*)o; a.lse = (float*)lse; a.d_o = d_o; a.dq = dq;
  a.kind = mode; a.window = window; a.block_size = block_size;
  if (mode == NSA_MODE_COMPRESS) a.window = block_size;   // internally `window` holds the summary stride
  if (mode == NSA_MODE_COMPRESS_STRIDED) {
    NSA_CHECK_ARG(window >= 1 && window <= block_size, "summary stride must be in [1, block_size]");
    a.kind = NSA_MODE_COMPRESS;
  }
  a.row_scale = row_scale; a.row_dot = row_dot;
  a.dq_acc = dq_acc;
  NSA_CHECK_ARG((row_scale == nullptr) == (row_dot == nullptr), "row_scale and row_dot go together");
  if (use_tc(dims, 64, impl, &rc)) {
    a.dk_acc = (float*)dk;   // tc path writes dk/dv itself; pass the outputs through
    a.dv_acc = (float*)dv;
    return tc_attn_bwd(a, workspace, workspace_bytes, st);
  }
  if (rc != NSA_OK) return rc;
  NSA_CHECK_ARG(!dq_acc, "the dQ accumulator needs a shape the tcgen05 kernels serve");
  NSA_CHECK_ARG(dq, "dq may be null only when the tcgen05 kernels serve the call");
  return simt_bwd(a, dims, dk, dv, workspace, workspace_bytes, st);
}

extern "C" int nsa_range_attn_bwd(const void* q, const void* k, const void* v, const void* o,
                                  const float* lse, const void* d_o, void* dq, void* dk, void* dv,
                                  const NsaDims* dims, int Lk, int mode, int window, int block_size,
                                  const float* row_scale, const float* row_dot,
                                  void* workspace, size_t workspace_bytes, int impl, void* stream) {
  return range_attn_bwd(q, k, v, o, lse, d_o, dq, nullptr, dk, dv, dims, Lk, mode, window, block_size,
                        row_scale, row_dot, workspace, workspace_bytes, impl, stream);
}

extern "C" int nsa_range_attn_bwd_acc(const void* q, const void* k, const void* v, const void* o,
                                      const float* lse, const void* d_o, float* dq_acc, void* dk, void* dv,
                                      const NsaDims* dims, int Lk, int mode, int window, int block_size,
                                      const float* row_scale, const float* row_dot,
                                      void* workspace, size_t workspace_bytes, void* stream) {
  NSA_CHECK_ARG(dq_acc, "null dq accumulator");
  return range_attn_bwd(q, k, v, o, lse, d_o, nullptr, dq_acc, dk, dv, dims, Lk, mode, window, block_size,
                        row_scale, row_dot, workspace, workspace_bytes, NSA_IMPL_TC, stream);
}

// ---- selection attention ---------------------------------------------------------------------
extern "C" size_t nsa_selection_fwd_workspace_bytes(const NsaDims* dims, int S, int block_size,
                                                    int impl) {
  if (check_dims(dims) != NSA_OK || S <= 0) return 0;
  int rc;
  if (!use_tc(dims, block_size, impl, &rc)) return 0;
  AttnArgs a = base_args(dims, dims->T);
  a.kind = 2; a.S = S; a.block_size = block_size;
  return tc_sel_fwd_workspace(a);
}

static int check_sel(const NsaDims* dims, int S, int block_size) {
  int rc = check_dims(dims);
  if (rc != NSA_OK) return rc;
  NSA_CHECK_ARG(S >= 0, "bad S");
  NSA_CHECK_ARG(block_size >= 16, "block_size must be >= 16");   // nsa_selection_kernel.py:188
  return NSA_OK;
}

static int selection_fwd_impl(const void* q, const void* k, const void* v,
                              const int32_t* block_idx, void* o, float* lse, const NsaDims* dims,
                              int S, int block_size, void* workspace, size_t workspace_bytes,
                              int impl, const void* plan, void* stream);

extern "C" int nsa_selection_fwd(const void* q, const void* k, const void* v,
                                 const int32_t* block_idx, void* o, float* lse, const NsaDims* dims,
                                 int S, int block_size, void* workspace, size_t workspace_bytes,
                                 int impl, void* stream) {
  return selection_fwd_impl(q, k, v, block_idx, o, lse, dims, S, block_size, workspace, workspace_bytes, impl,
                            nullptr, stream);
}

extern "C" int nsa_selection_fwd_planned(const void* q, const void* k, const void* v,
                                         const int32_t* block_idx, void* o, float* lse, const NsaDims* dims,
                                         int S, int block_size, void* workspace, size_t workspace_bytes,
                                         const void* plan, void* stream) {
  NSA_CHECK_ARG(plan, "null plan");
  return selection_fwd_impl(q, k, v, block_idx, o, lse, dims, S, block_size, workspace, workspace_bytes,
                            NSA_IMPL_TC, plan, stream);
}

static int selection_fwd_impl(const void* q, const void* k, const void* v,
                              const int32_t* block_idx, void* o, float* lse, const NsaDims* dims,
                              int S, int block_size, void* workspace, size_t workspace_bytes,
                              int impl, const void* plan, void* stream) {
  int rc = check_sel(dims, S, block_size);
  if (rc != NSA_OK) return rc;
  const size_t rows = (size_t)dims->B * dims->Hq * dims->T;
  if (rows == 0) return NSA_OK;
  NSA_CHECK_ARG(q && k && v && o && lse && (S == 0 || block_idx), "null tensor");
  AttnArgs a = base_args(dims, dims->T);
  a.q = q; a.k = k; a.v = v; a.o = o; a.lse = lse; a.block_idx = block_idx;
  a.kind = 2; a.S = S; a.block_size = block_size;
  a.sel_plan = plan;
  if (use_tc(dims, block_size, impl, &rc) && S > 0)
    return tc_sel_fwd(a, workspace, workspace_bytes, (cudaStream_t)stream);
  if (rc != NSA_OK) return rc;
  return simt_attn_fwd(a, dims->dtype, (cudaStream_t)stream);
}

extern "C" size_t nsa_selection_plan_bytes(const NsaDims* dims, int S, int block_size) {
  if (check_sel(dims, S, block_size) != NSA_OK || S <= 0) return 0;
  int rc;
  if (!use_tc(dims, block_size, NSA_IMPL_AUTO, &rc)) return 0;
  AttnArgs a = base_args(dims, dims->T);
  a.kind = 2; a.S = S; a.block_size = block_size;
  return tc_sel_plan_bytes(a);
}

extern "C" int nsa_selection_plan_build(const int32_t* block_idx, const NsaDims* dims, int S, int block_size,
                                        void* plan, size_t plan_bytes, void* stream) {
  int rc = check_sel(dims, S, block_size);
  if (rc != NSA_OK) return rc;
  NSA_CHECK_ARG(S > 0 && block_idx && plan, "null block_idx or plan");
  NSA_CHECK_ARG(use_tc(dims, block_size, NSA_IMPL_AUTO, &rc), "a selection plan needs a shape the tcgen05 kernels serve");
  AttnArgs a = base_args(dims, dims->T);
  a.block_idx = block_idx; a.kind = 2; a.S = S; a.block_size = block_size;
  return tc_sel_plan_build(a, plan, plan_bytes, (cudaStream_t)stream);
}

extern "C" size_t nsa_selection_bwd_workspace_bytes(const NsaDims* dims, int S, int block_size,
                                                    int impl) {
  if (check_sel(dims, S, block_size) != NSA_OK) return 0;
  int rc;
  size_t need = simt_bwd_ws(dims, dims->T);
  if (use_tc(dims, block_size, impl, &rc)) {
    AttnArgs a = base_args(dims, dims->T);
    a.kind = 2; a.S = S; a.block_size = block_size;
    need = need > tc_attn_bwd_workspace(a) ? need : tc_attn_bwd_workspace(a);
  }
  return need;
}

static int selection_bwd_impl(const void* q, const void* k, const void* v,
                              const int32_t* block_idx, const void* o, const float* lse,
                              const void* d_o, void* dq, void* dk, void* dv, const NsaDims* dims,
                              int S, int block_size, const float* row_scale, const float* row_dot,
                              void* workspace, size_t workspace_bytes, int impl, const void* plan, void* stream);

extern "C" int nsa_selection_bwd(const void* q, const void* k, const void* v,
                                 const int32_t* block_idx, const void* o, const float* lse,
                                 const void* d_o, void* dq, void* dk, void* dv, const NsaDims* dims,
                                 int S, int block_size, const float* row_scale, const float* row_dot,
                                 void* workspace, size_t workspace_bytes, int impl, void* stream) {
  return selection_bwd_impl(q, k, v, block_idx, o, lse, d_o, dq, dk, dv, dims, S, block_size, row_scale, row_dot,
                            workspace, workspace_bytes, impl, nullptr, stream);
}

extern "C" int nsa_selection_bwd_planned(const void* q, const void* k, const void* v,
                                         const int32_t* block_idx, const void* o, const float* lse,
                                         const void* d_o, void* dq, void* dk, void* dv, const NsaDims* dims,
                                         int S, int block_size, const float* row_scale, const float* row_dot,
                                         void* workspace, size_t workspace_bytes, const void* plan, void* stream) {
  NSA_CHECK_ARG(plan, "null plan");
  return selection_bwd_impl(q, k, v, block_idx, o, lse, d_o, dq, dk, dv, dims, S, block_size, row_scale, row_dot,
                            workspace, workspace_bytes, NSA_IMPL_TC, plan, stream);
}

static int selection_bwd_impl(const void* q, const void* k, const void* v,
                              const int32_t* block_idx, const void* o, const float* lse,
                              const void* d_o, void* dq, void* dk, void* dv, const NsaDims* dims,
                              int S, int block_size, const float* row_scale, const float* row_dot,
                              void* workspace, size_t workspace_bytes, int impl, const void* plan, void* stream) {
  int rc = check_sel(dims, S, block_size);
  if (rc != NSA_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t rows = (size_t)dims->B * dims->Hq * dims->T;
  if (rows == 0) return NSA_OK;
  NSA_CHECK_ARG(q && k && v && o && lse && d_o && dk && dv && (S == 0 || block_idx),
                "null tensor");
  AttnArgs a = base_args(dims, dims->T);
  a.q = q; a.k = k; a.v = v; a.o = (void*)o; a.lse = (float*)lse; a.d_o = d_o; a.dq = dq;
  a.block_idx = block_idx; a.kind = 2; a.S = S; a.block_size = block_size;
  a.row_scale = row_scale; a.row_dot = row_dot;
  NSA_CHECK_ARG((row_scale == nullptr) == (row_dot == nullptr), "row_scale and row_dot go together");
  if (use_tc(dims, block_size, impl, &rc) && S > 0) {
    a.dk_acc = (float*)dk;
    a.dv_acc = (float*)dv;
    a.sel_plan = plan;
    return tc_attn_bwd(a, workspace, workspace_bytes, st);
  }
  if (rc != NSA_OK) return rc;
  NSA_CHECK_ARG(dq, "dq may be null only when the tcgen05 kernels serve the call");
  return simt_bwd(a, dims, dk, dv, workspace, workspace_bytes, st);
}

extern "C" int nsa_dq_reduce3(const NsaDims* dims, int Lk_cmp, int cmp_len, int cmp_stride, int S,
                              int block_size, int window, const void* ws_cmp, const void* ws_slc,
                              const void* ws_win, void* dq, void* stream) {
  int rc = check_dims(dims);
  if (rc != NSA_OK) return rc;
  NSA_CHECK_ARG(dq, "null dq");
  NSA_CHECK_ARG(use_tc(dims, block_size, NSA_IMPL_AUTO, &rc), "nsa_dq_reduce3 needs a shape the tcgen05 kernels serve");
  if (cmp_stride <= 0) cmp_stride = cmp_len;
  NSA_CHECK_ARG(!ws_cmp || (Lk_cmp > 0 && cmp_len > 0 && cmp_stride <= cmp_len), "bad compression geometry");
  NSA_CHECK_ARG(!ws_slc || S > 0, "bad S");
  NSA_CHECK_ARG(!ws_win || window >= 1, "bad window");
  const AttnArgs a = base_args(dims, dims->T);
  return tc_dq_reduce3(a, Lk_cmp, cmp_len, cmp_stride, S, block_size, window, ws_cmp, ws_slc, ws_win,
                       nullptr, dq, (cudaStream_t)stream);
}

extern "C" int nsa_dq_finish(const NsaDims* dims, int S, int block_size, const float* dq_acc,
                             const void* ws_slc, void* dq, void* stream) {
  int rc = check_dims(dims);
  if (rc != NSA_OK) return rc;
  NSA_CHECK_ARG(dq && dq_acc, "null dq or accumulator");
  NSA_CHECK_ARG(use_tc(dims, block_size, NSA_IMPL_AUTO, &rc), "nsa_dq_finish needs a shape the tcgen05 kernels serve");
  NSA_CHECK_ARG(!ws_slc || S > 0, "bad S");
  const AttnArgs a = base_args(dims, dims->T);
  return tc_dq_reduce3(a, 0, 0, 0, S, block_size, 1, nullptr, ws_slc, nullptr, dq_acc, dq, (cudaStream_t)stream);
}
