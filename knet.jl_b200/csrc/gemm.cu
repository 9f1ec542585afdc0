// Matrix products behind the knet_gemm_* entry points: the library call Knet makes for `*`,
// A_mul_Bt and At_mul_B of KnetMatrix (src/knetarrays/linalg.jl:11-55, cublasSgemm_v2 /
// cublasDgemm_v2 through CUDA.jl).  Only host code here: the products are cuBLAS kernels.
//
// cuBLAS is not a link-time dependency: it is opened with dlopen when the first handle is
// created (KNET_SM100_CUBLAS_LIB, else libcublas.so.12 - which is the copy a host such as
// PyTorch has already loaded, if any).  A handle belongs to its creator (one per host thread
// and device, as CUDA.jl's task-local CUBLAS.handle()); nothing is cached in globals besides
// the function table.
//
// Float32 products take a mode: 0 is cuBLAS's plain FP32 arithmetic (what the reference
// runs), 1 asks for cuBLAS's FP32 emulation on the BF16 tensor cores (every operand is
// split into three BF16 terms and the nine partial products are accumulated in FP32;
// offered by cuBLAS 12.9 and later) and answers KN_EUNSUPPORTED when the loaded cuBLAS
// is older.
#include <dlfcn.h>

#include <cstdlib>
#include <mutex>

#include "common.cuh"

#if __has_include(<cublas_v2.h>)
#include <cublas_v2.h>
#define KN_HAVE_CUBLAS_HEADER 1
#else
#define KN_HAVE_CUBLAS_HEADER 0
#endif

namespace kn {

enum : int { KN_ECUBLAS = -7, KN_EUNSUPPORTED = -8 };

#if KN_HAVE_CUBLAS_HEADER

struct CublasApi {
  void* lib = nullptr;
  decltype(&cublasCreate_v2) Create = nullptr;
  decltype(&cublasDestroy_v2) Destroy = nullptr;
  decltype(&cublasGetVersion_v2) GetVersion = nullptr;
  decltype(&cublasSetStream_v2) SetStream = nullptr;
  decltype(&cublasSetWorkspace_v2) SetWorkspace = nullptr;
  decltype(&cublasSetMathMode) SetMathMode = nullptr;
  cublasStatus_t (*GemmEx64)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int64_t, int64_t, int64_t,
                             const void*, const void*, cudaDataType, int64_t, const void*, cudaDataType, int64_t,
                             const void*, void*, cudaDataType, int64_t, cublasComputeType_t, cublasGemmAlgo_t) = nullptr;
  // present from cuBLAS 12.9 on
  cublasStatus_t (*SetEmulationStrategy)(cublasHandle_t, int) = nullptr;
  bool ok = false;
};

template <typename F> bool csym(void* h, const char* name, F& out) {
  out = reinterpret_cast<F>(dlsym(h, name));
  return out != nullptr;
}

CublasApi& cublas() {
  static CublasApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[3] = {getenv("KNET_SM100_CUBLAS_LIB"), "libcublas.so.12", "libcublas.so"};
    for (const char* n : names) {
      if (!n || !*n) continue;
      api.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (api.lib) break;
    }
    if (!api.lib) return;
    void* h = api.lib;
    api.ok = csym(h, "cublasCreate_v2", api.Create) && csym(h, "cublasDestroy_v2", api.Destroy) &&
             csym(h, "cublasGetVersion_v2", api.GetVersion) && csym(h, "cublasSetStream_v2", api.SetStream) &&
             csym(h, "cublasSetWorkspace_v2", api.SetWorkspace) && csym(h, "cublasSetMathMode", api.SetMathMode) &&
             csym(h, "cublasGemmEx_64", api.GemmEx64);
    csym(h, "cublasSetEmulationStrategy", api.SetEmulationStrategy);
  });
  return api;
}

struct Gemm {
  cublasHandle_t h;
  int version;       // cublasGetVersion: 10000*major + 100*minor + patch
  int strategy;      // emulation strategy last given to the handle (-1: none yet)
};

inline int cublas_status(cublasStatus_t r) { return r == CUBLAS_STATUS_SUCCESS ? KN_OK : 2000 + (int)r; }
inline bool emulation_offered(const Gemm* g) { return g->version >= 120900; }

inline bool op_ok(int t) { return t == 0 || t == 1; }

// C (m,n) = alpha * op(A) (m,k) * op(B) (k,n) + beta * C, column-major.
template <typename T>
int gemm_run(void* handle, int ta, int tb, int64_t m, int64_t n, int64_t k, T alpha, const T* A, int64_t lda,
             const T* B, int64_t ldb, T beta, T* C, int64_t ldc, int mode, void* ws, size_t ws_bytes,
             cudaStream_t st) {
  Gemm* g = static_cast<Gemm*>(handle);
  constexpr bool f32 = sizeof(T) == 4;
  if (!g || !op_ok(ta) || !op_ok(tb) || m < 0 || n < 0 || k < 0) return KN_EINVAL;
  if (mode < 0 || mode > 2 || (!f32 && mode != 0)) return KN_EINVAL;
  if (m == 0 || n == 0) return KN_OK;
  if (!C || ldc < m) return KN_EINVAL;
  if (k > 0 && (!A || !B || lda < (ta ? k : m) || ldb < (tb ? n : k))) return KN_EINVAL;
  if ((ws == nullptr) != (ws_bytes == 0) || ((uintptr_t)ws & 255)) return KN_EINVAL;
  if (!cublas().ok) return KN_ECUBLAS;
  if (mode != 0 && !emulation_offered(g)) return KN_EUNSUPPORTED;
  cublasStatus_t r = cublas().SetStream(g->h, st);
  if (r != CUBLAS_STATUS_SUCCESS) return cublas_status(r);
  if (ws) {
    r = cublas().SetWorkspace(g->h, ws, ws_bytes);
    if (r != CUBLAS_STATUS_SUCCESS) return cublas_status(r);
  }
  cublasComputeType_t ct = f32 ? CUBLAS_COMPUTE_32F : CUBLAS_COMPUTE_64F;
  if (mode != 0) {
    // 1: emulate whenever cuBLAS can; 2: leave the choice to cuBLAS's own heuristics
    const int want = mode == 1 ? (int)CUBLAS_EMULATION_STRATEGY_EAGER : (int)CUBLAS_EMULATION_STRATEGY_PERFORMANT;
    if (g->strategy != want) {
      if (!cublas().SetEmulationStrategy) return KN_EUNSUPPORTED;
      r = cublas().SetEmulationStrategy(g->h, want);
      if (r != CUBLAS_STATUS_SUCCESS) return cublas_status(r);
      g->strategy = want;
    }
    ct = CUBLAS_COMPUTE_32F_EMULATED_16BFX9;
  }
  const cudaDataType dt = f32 ? CUDA_R_32F : CUDA_R_64F;
  r = cublas().GemmEx64(g->h, ta ? CUBLAS_OP_T : CUBLAS_OP_N, tb ? CUBLAS_OP_T : CUBLAS_OP_N, m, n, k, &alpha, A, dt,
                        lda, B, dt, ldb, &beta, C, dt, ldc, ct, CUBLAS_GEMM_DEFAULT);
  return cublas_status(r);
}

#endif  // KN_HAVE_CUBLAS_HEADER

}  // namespace kn

using namespace kn;

#if KN_HAVE_CUBLAS_HEADER

KN_EXPORT int knet_gemm_create(void** handle) {
  if (!handle) return KN_EINVAL;
  if (!cublas().ok) return KN_ECUBLAS;
  Gemm* g = new Gemm{nullptr, 0, -1};
  cublasStatus_t r = cublas().Create(&g->h);
  if (r != CUBLAS_STATUS_SUCCESS) {
    delete g;
    return cublas_status(r);
  }
  // plain FP32 arithmetic unless a call asks otherwise: no TF32, whatever the environment's default
  cublas().SetMathMode(g->h, CUBLAS_DEFAULT_MATH);
  r = cublas().GetVersion(g->h, &g->version);
  if (r != CUBLAS_STATUS_SUCCESS) g->version = 0;
  *handle = g;
  return KN_OK;
}

KN_EXPORT int knet_gemm_destroy(void* handle) {
  Gemm* g = static_cast<Gemm*>(handle);
  if (!g) return KN_EINVAL;
  const cublasStatus_t r = cublas().ok ? cublas().Destroy(g->h) : CUBLAS_STATUS_NOT_INITIALIZED;
  delete g;
  return cublas_status(r);
}

KN_EXPORT int knet_gemm_version(void* handle) {
  Gemm* g = static_cast<Gemm*>(handle);
  return g ? g->version : KN_EINVAL;
}

KN_EXPORT int knet_gemm_emulation(void* handle) {
  Gemm* g = static_cast<Gemm*>(handle);
  if (!g) return KN_EINVAL;
  return (emulation_offered(g) && cublas().SetEmulationStrategy) ? 1 : 0;
}

KN_EXPORT int knet_gemm_32_S(void* handle, int transA, int transB, int64_t m, int64_t n, int64_t k, float alpha,
                             const float* A, int64_t lda, const float* B, int64_t ldb, float beta, float* C,
                             int64_t ldc, int mode, void* workspace, size_t workspace_bytes, cudaStream_t s) {
  return gemm_run<float>(handle, transA, transB, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, mode, workspace,
                         workspace_bytes, s);
}

KN_EXPORT int knet_gemm_64_S(void* handle, int transA, int transB, int64_t m, int64_t n, int64_t k, double alpha,
                             const double* A, int64_t lda, const double* B, int64_t ldb, double beta, double* C,
                             int64_t ldc, int mode, void* workspace, size_t workspace_bytes, cudaStream_t s) {
  return gemm_run<double>(handle, transA, transB, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, mode, workspace,
                          workspace_bytes, s);
}

#else  // no cuBLAS header at build time: the entry points exist and say so

KN_EXPORT int knet_gemm_create(void**) { return KN_ECUBLAS; }
KN_EXPORT int knet_gemm_destroy(void*) { return KN_ECUBLAS; }
KN_EXPORT int knet_gemm_version(void*) { return KN_ECUBLAS; }
KN_EXPORT int knet_gemm_emulation(void*) { return KN_ECUBLAS; }
KN_EXPORT int knet_gemm_32_S(void*, int, int, int64_t, int64_t, int64_t, float, const float*, int64_t, const float*,
                             int64_t, float, float*, int64_t, int, void*, size_t, cudaStream_t) {
  return KN_ECUBLAS;
}
KN_EXPORT int knet_gemm_64_S(void*, int, int, int64_t, int64_t, int64_t, double, const double*, int64_t,
                             const double*, int64_t, double, double*, int64_t, int, void*, size_t, cudaStream_t) {
  return KN_ECUBLAS;
}

#endif
