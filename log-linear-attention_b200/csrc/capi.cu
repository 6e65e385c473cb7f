// extern "C" entry points of libllattn.so: argument checks, workspace carving, launches.
#include <stdint.h>

#include "llattn_gdn.h"
#include "llattn_mamba2.h"
#include "llattn_testing.h"

namespace llattn {
std::atomic<unsigned long long> g_kernel_launches{0};
}

namespace {

inline size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

struct Carver {
    unsigned char* base;
    size_t off;
    explicit Carver(void* p) : base(reinterpret_cast<unsigned char*>(p)), off(0) {}
    template <typename T>
    T* take(size_t count) {
        T* r = base ? reinterpret_cast<T*>(base + off) : nullptr;
        off += align_up(count * sizeof(T));
        return r;
    }
};

int ceil_log2i(int x) {
    int l = 0;
    while ((1 << l) < x) ++l;
    return l;
}

int check_shape(int B, int T, int H, int G, int K, int V, int L) {
    if (B <= 0 || T <= 0 || H <= 0 || G <= 0) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (T % llattn_chunk() != 0) return LLATTN_ERR_BAD_LENGTH;
    if (H % G != 0) return LLATTN_ERR_BAD_GROUPS;
    if (!((K == 64 || K == 128) && V == 64)) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (L > 32) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (L < 7 + ceil_log2i(T / 64)) return LLATTN_ERR_TOO_FEW_LEVELS;
    // the per-level scans over segments hold at most M2_MAX_LH segment levels: T <= 512 * 2^10 tokens
    const int seg = 1 << llattn::M2_MLOW;
    if (ceil_log2i((T / 64 + seg - 1) / seg) > llattn::M2_MAX_LH) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    return 0;
}

// fills the size-dependent fields and carves the scratch buffers (base may be NULL to size only)
size_t setup(llattn::Mamba2Params& p, void* ws, bool backward) {
    const int SEG = 1 << llattn::M2_MLOW;
    p.NT = p.T / 64;
    p.NS = (p.NT + SEG - 1) / SEG;
    p.LH = ceil_log2i(p.NS);
    p.o_has_high = p.NS > 1;
    p.LZ = llattn::M2_MLOW + p.LH;
    const size_t KV = (size_t)p.K * p.V, BH = (size_t)p.B * p.H;
    Carver c(ws);
    p.err = c.take<int>(64);      // status word first (256 bytes)
    if (p.NS > 1) {
        p.seg_F = c.take<float>(BH * p.NS * KV);
        p.seg_D = c.take<float>(BH * p.NS);
        p.seg_H0 = c.take<__nv_bfloat16>(BH * p.NS * p.LH * KV);
        p.o_hi = c.take<__nv_bfloat16>((size_t)p.B * p.T * p.H * p.V);
    }
    if (backward) {
        p.g = c.take<float>((size_t)p.B * p.T * p.H);
        p.dq_acc = c.take<float>((size_t)p.B * p.T * p.G * p.K);
        p.dk_acc = c.take<float>((size_t)p.B * p.T * p.G * p.K);
        p.wq = c.take<float>((size_t)p.B * p.T * p.H);
        p.Yseg = c.take<float>(BH * p.NS * (p.LH > 0 ? p.LH : 1));
        p.Zc = c.take<float>(BH * p.NT * p.LZ);
        p.Yc = c.take<float>(BH * p.NT * (llattn::M2_MLOW + 1));
        if (p.NS > 1) {
            p.seg_dF = c.take<float>(BH * p.NS * p.LH * KV);
            p.seg_dHf = c.take<float>(BH * p.NS * KV);
        }
    }
    return c.off;
}

// Scratch for llattn_mamba2_fwd_static.  The array lives in the library's device image: every GPU
// that loads the library carries these bytes until the process exits.  In host code the symbol is
// only a handle; the device address is obtained once per device with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[LLATTN_STATIC_SCRATCH_BYTES];
static void* g_static_scratch_addr[64] = {nullptr};

}  // namespace

extern "C" {

int llattn_version(void) { return 2; }
void llattn_testing_use_tensor_core_path(int enabled) { llattn::g_use_tensor_core_path.store(enabled ? 1 : 0); }
unsigned long long llattn_kernel_launches(void) { return llattn::g_kernel_launches.load(); }

int llattn_workspace_status(const void* workspace, int* status_host, void* stream) {
    if (!workspace || !status_host) return LLATTN_ERR_NULL;
    cudaError_t e = cudaMemcpyAsync(status_host, workspace, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    return (int)cudaStreamSynchronize((cudaStream_t)stream);
}
int llattn_chunk(void) { return 64; }

size_t llattn_mamba2_fwd_workspace_bytes(int B, int T, int H, int G, int K, int V, int L) {
    if (check_shape(B, T, H, G, K, V, L) != 0) return 0;
    llattn::Mamba2Params p = {};
    p.B = B; p.T = T; p.H = H; p.G = G; p.K = K; p.V = V; p.L = L;
    return setup(p, nullptr, false);
}

int llattn_mamba2_fwd(const void* q, const void* k, const void* v, const float* g, const void* lambda,
                      void* o, float* g_cum, void* workspace, size_t workspace_bytes,
                      int B, int T, int H, int G, int K, int V, int L, void* stream) {
    int rc = check_shape(B, T, H, G, K, V, L);
    if (rc != 0) return rc;
    if (!q || !k || !v || !g || !lambda || !o || !g_cum) return LLATTN_ERR_NULL;
    llattn::Mamba2Params p = {};
    p.B = B; p.T = T; p.H = H; p.G = G; p.K = K; p.V = V; p.L = L;
    const size_t need = setup(p, nullptr, false);
    if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255)) return LLATTN_ERR_WORKSPACE;
    setup(p, workspace, false);
    p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v;
    p.g = g; p.l = (const __nv_bfloat16*)lambda;
    p.o = (__nv_bfloat16*)o; p.g_cum = g_cum;
    cudaError_t e = cudaMemsetAsync(p.err, 0, sizeof(int), (cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    return llattn::mamba2_fwd_dispatch(p, (cudaStream_t)stream);
}

size_t llattn_static_scratch_bytes(void) { return LLATTN_STATIC_SCRATCH_BYTES; }

int llattn_static_scratch_status(int* status_host, void* stream) {
    if (!status_host) return LLATTN_ERR_NULL;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (g_static_scratch_addr[dev] == nullptr) {   // no call has used the array on this device yet
        *status_host = 0;
        return 0;
    }
    return llattn_workspace_status(g_static_scratch_addr[dev], status_host, stream);
}

int llattn_mamba2_fwd_static(const void* q, const void* k, const void* v, const float* g, const void* lambda,
                             void* o, float* g_cum, int B, int T, int H, int G, int K, int V, int L, void* stream) {
    int rc = check_shape(B, T, H, G, K, V, L);
    if (rc != 0) return rc;
    if (!q || !k || !v || !g || !lambda || !o || !g_cum) return LLATTN_ERR_NULL;
    llattn::Mamba2Params p = {};
    p.B = B; p.T = T; p.H = H; p.G = G; p.K = K; p.V = V; p.L = L;
    const size_t need = setup(p, nullptr, false);
    if (need > (size_t)LLATTN_STATIC_SCRATCH_BYTES) return LLATTN_ERR_STATIC_SCRATCH;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (g_static_scratch_addr[dev] == nullptr) {
        // first call on this device (it is the current one): resolve the device address of the array
        void* addr = nullptr;
        e = cudaGetSymbolAddress(&addr, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (addr == nullptr) return LLATTN_ERR_WORKSPACE;
        g_static_scratch_addr[dev] = addr;
    }
    // every scratch element that a kernel reads is written earlier in the same call, so nothing
    // has to be cleared even though the previous call's contents are still there
    setup(p, g_static_scratch_addr[dev], false);
    p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v;
    p.g = g; p.l = (const __nv_bfloat16*)lambda;
    p.o = (__nv_bfloat16*)o; p.g_cum = g_cum;
    e = cudaMemsetAsync(p.err, 0, sizeof(int), (cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    return llattn::mamba2_fwd_dispatch(p, (cudaStream_t)stream);
}

size_t llattn_mamba2_bwd_workspace_bytes(int B, int T, int H, int G, int K, int V, int L) {
    if (check_shape(B, T, H, G, K, V, L) != 0) return 0;
    llattn::Mamba2Params p = {};
    p.B = B; p.T = T; p.H = H; p.G = G; p.K = K; p.V = V; p.L = L;
    return setup(p, nullptr, true);
}

int llattn_mamba2_bwd(const void* q, const void* k, const void* v, const float* g_cum, const void* lambda,
                      const void* d_o, void* dq, void* dk, void* dv, float* dg, float* dlambda,
                      void* workspace, size_t workspace_bytes,
                      int B, int T, int H, int G, int K, int V, int L, void* stream) {
    return llattn_mamba2_bwd_saved(q, k, v, g_cum, lambda, d_o, dq, dk, dv, dg, dlambda, workspace, workspace_bytes,
                                   nullptr, 0, B, T, H, G, K, V, L, stream);
}

int llattn_mamba2_bwd_saved(const void* q, const void* k, const void* v, const float* g_cum, const void* lambda,
                            const void* d_o, void* dq, void* dk, void* dv, float* dg, float* dlambda,
                            void* workspace, size_t workspace_bytes, const void* fwd_workspace, size_t fwd_workspace_bytes,
                            int B, int T, int H, int G, int K, int V, int L, void* stream) {
    int rc = check_shape(B, T, H, G, K, V, L);
    if (rc != 0) return rc;
    if (!q || !k || !v || !g_cum || !lambda || !d_o || !dq || !dk || !dv || !dg || !dlambda) return LLATTN_ERR_NULL;
    llattn::Mamba2Params p = {};
    p.B = B; p.T = T; p.H = H; p.G = G; p.K = K; p.V = V; p.L = L;
    const size_t need = setup(p, nullptr, true);
    if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255)) return LLATTN_ERR_WORKSPACE;
    setup(p, workspace, true);
    if (fwd_workspace) {
        // segment decays and level states as the forward call left them in its workspace
        llattn::Mamba2Params pf = {};
        pf.B = B; pf.T = T; pf.H = H; pf.G = G; pf.K = K; pf.V = V; pf.L = L;
        const size_t fneed = setup(pf, nullptr, false);
        if (fwd_workspace_bytes < fneed || ((uintptr_t)fwd_workspace & 255)) return LLATTN_ERR_WORKSPACE;
        setup(pf, const_cast<void*>(fwd_workspace), false);
        p.seg_F = pf.seg_F; p.seg_D = pf.seg_D; p.seg_H0 = pf.seg_H0;
        p.reuse_states = 1;
    }
    cudaStream_t st = (cudaStream_t)stream;
    p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v;
    p.l = (const __nv_bfloat16*)lambda; p.d_o = (const __nv_bfloat16*)d_o;
    p.dv = (__nv_bfloat16*)dv; p.dl = dlambda;
    const size_t nqk = (size_t)B * T * G * K, nbth = (size_t)B * T * H;
    cudaError_t e;
    if ((e = cudaMemsetAsync(p.err, 0, sizeof(int), st)) != cudaSuccess) return (int)e;
    // dq_acc, dk_acc, wq and Yseg are adjacent in the workspace: one clear covers the four
    if ((e = cudaMemsetAsync(p.dq_acc, 0, (size_t)((unsigned char*)p.Zc - (unsigned char*)p.dq_acc), st)) != cudaSuccess) return (int)e;
    if ((e = cudaMemsetAsync(dlambda, 0, nbth * L * sizeof(float), st)) != cudaSuccess) return (int)e;
    llattn::mamba2_uncumsum(g_cum, const_cast<float*>(p.g), (long)B * T, H, st);
    rc = llattn::mamba2_bwd_dispatch(p, st);
    if (rc != 0) return rc;
    if ((rc = llattn::mamba2_dg(p, dg, st)) != 0) return rc;
    llattn::cast_f32_to_bf16(p.dq_acc, dq, (long)nqk, st);
    llattn::cast_f32_to_bf16(p.dk_acc, dk, (long)nqk, st);
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- Gated DeltaNet
static int gdn_check(int B, int T, int H, int K, int V, int L) {
    if (B <= 0 || T <= 0 || H <= 0) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (T % 64 != 0) return LLATTN_ERR_BAD_LENGTH;
    if (!(K == 128 && (V == 64 || V == 128))) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (L > 32) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    const int nlev = ceil_log2i(T / 64);
    if (nlev > 8) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (L < 7 + nlev) return LLATTN_ERR_TOO_FEW_LEVELS;
    return 0;
}

// workspace parts: chunk matrices (kd, wd, qd, u), level states hs, adjoint level states dhs
enum { GDN_WS_CHUNK = 1, GDN_WS_HS = 2, GDN_WS_DHS = 4 };
static size_t gdn_setup(llattn::GdnParams& p, void* ws, int parts, size_t start = 0) {
    p.NT = p.T / 64;
    p.NLEV = ceil_log2i(p.NT);
    Carver c(ws);
    c.off = start;
    p.err = c.take<int>(64);      // status word first (256 bytes)
    const size_t n = (size_t)p.B * p.T * p.H;
    if (parts & GDN_WS_CHUNK) {
        p.kd = c.take<__nv_bfloat16>(n * p.K);
        p.wd = c.take<__nv_bfloat16>(n * p.K);
        p.qd = c.take<__nv_bfloat16>(n * p.K);
        p.u = c.take<__nv_bfloat16>(n * p.V);
        p.wk = c.take<__nv_bfloat16>((size_t)p.B * p.NT * p.H * p.K * p.K);
    }
    // level states and their adjoints: one K x 32 tile per (batch, head, 32-column slice, chunk, level)
    const size_t tiles = (size_t)p.B * p.H * (p.V / llattn::GDN_VS) * p.NT * (p.NLEV > 0 ? p.NLEV : 1);
    if (parts & GDN_WS_HS) p.hs = c.take<__nv_bfloat16>(tiles * p.K * llattn::GDN_VS);
    if (parts & GDN_WS_DHS) p.dhs = c.take<__nv_bfloat16>(tiles * p.K * llattn::GDN_VS);
    return c.off;
}

size_t llattn_gdn_fwd_workspace_bytes(int B, int T, int H, int K, int V, int L) {
    if (gdn_check(B, T, H, K, V, L) != 0) return 0;
    llattn::GdnParams p = {};
    p.B = B; p.T = T; p.H = H; p.K = K; p.V = V; p.L = L;
    return gdn_setup(p, nullptr, GDN_WS_CHUNK);
}

size_t llattn_gdn_fwd_keep_workspace_bytes(int B, int T, int H, int K, int V, int L) {
    if (gdn_check(B, T, H, K, V, L) != 0) return 0;
    llattn::GdnParams p = {};
    p.B = B; p.T = T; p.H = H; p.K = K; p.V = V; p.L = L;
    return gdn_setup(p, nullptr, GDN_WS_CHUNK | GDN_WS_HS);
}

static int gdn_fwd_impl(const void* q, const void* k, const void* v, const void* beta, const float* g, const void* lambda,
                        void* o, float* g_cum, void* Aw, void* Au, void* workspace, size_t workspace_bytes,
                        int B, int T, int H, int K, int V, int L, void* stream, bool keep, float* final_states = nullptr);

int llattn_gdn_prefill(const void* q, const void* k, const void* v, const void* beta, const float* g, const void* lambda,
                       void* o, float* g_cum, void* Aw, void* Au, float* states, void* workspace, size_t workspace_bytes,
                       int B, int T, int H, int K, int V, int L, void* stream) {
    if (!states) return LLATTN_ERR_NULL;
    int rc = gdn_check(B, T, H, K, V, L);
    if (rc != 0) return rc;
    cudaError_t e = cudaMemsetAsync(states, 0, (size_t)B * H * K * V * L * sizeof(float), (cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    return gdn_fwd_impl(q, k, v, beta, g, lambda, o, g_cum, Aw, Au, workspace, workspace_bytes, B, T, H, K, V, L, stream, false, states);
}

int llattn_gdn_fwd(const void* q, const void* k, const void* v, const void* beta, const float* g, const void* lambda,
                   void* o, float* g_cum, void* Aw, void* Au, void* workspace, size_t workspace_bytes,
                   int B, int T, int H, int K, int V, int L, void* stream) {
    return gdn_fwd_impl(q, k, v, beta, g, lambda, o, g_cum, Aw, Au, workspace, workspace_bytes, B, T, H, K, V, L, stream, false);
}

int llattn_gdn_fwd_keep(const void* q, const void* k, const void* v, const void* beta, const float* g, const void* lambda,
                        void* o, float* g_cum, void* Aw, void* Au, void* workspace, size_t workspace_bytes,
                        int B, int T, int H, int K, int V, int L, void* stream) {
    return gdn_fwd_impl(q, k, v, beta, g, lambda, o, g_cum, Aw, Au, workspace, workspace_bytes, B, T, H, K, V, L, stream, true);
}

static int gdn_fwd_impl(const void* q, const void* k, const void* v, const void* beta, const float* g, const void* lambda,
                        void* o, float* g_cum, void* Aw, void* Au, void* workspace, size_t workspace_bytes,
                        int B, int T, int H, int K, int V, int L, void* stream, bool keep, float* final_states) {
    int rc = gdn_check(B, T, H, K, V, L);
    if (rc != 0) return rc;
    if (!q || !k || !v || !beta || !g || !lambda || !o || !g_cum || !Aw || !Au) return LLATTN_ERR_NULL;
    llattn::GdnParams p = {};
    p.B = B; p.T = T; p.H = H; p.K = K; p.V = V; p.L = L;
    const int parts = keep ? (GDN_WS_CHUNK | GDN_WS_HS) : GDN_WS_CHUNK;
    const size_t need = gdn_setup(p, nullptr, parts);
    if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255)) return LLATTN_ERR_WORKSPACE;
    gdn_setup(p, workspace, parts);
    p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v;
    p.beta = (const __nv_bfloat16*)beta; p.g = g; p.l = (const __nv_bfloat16*)lambda;
    p.o = (__nv_bfloat16*)o; p.g_cum = g_cum; p.Aw = (__nv_bfloat16*)Aw; p.Au = (__nv_bfloat16*)Au;
    p.final_states = final_states;
    cudaError_t e0 = cudaMemsetAsync(p.err, 0, sizeof(int), (cudaStream_t)stream);
    if (e0 != cudaSuccess) return (int)e0;
    return keep ? llattn::gdn_fwd_keep_dispatch(p, (cudaStream_t)stream) : llattn::gdn_fwd_dispatch(p, (cudaStream_t)stream);
}

size_t llattn_gdn_bwd_levels_workspace_bytes(int B, int T, int H, int K, int V, int L) {
    if (gdn_check(B, T, H, K, V, L) != 0) return 0;
    llattn::GdnParams p = {};
    p.B = B; p.T = T; p.H = H; p.K = K; p.V = V; p.L = L;
    return gdn_setup(p, nullptr, GDN_WS_CHUNK | GDN_WS_HS | GDN_WS_DHS);
}

int llattn_gdn_bwd_levels(const void* q, const void* k, const void* v, const void* beta, const float* g_cum, const void* lambda,
                          const void* Aw, const void* Au, const void* d_o, float* d_qd, float* d_wd, float* d_kd, void* d_u,
                          float* d_gl, float* dlambda, void* workspace, size_t workspace_bytes,
                          int B, int T, int H, int K, int V, int L, void* stream) {
    int rc = gdn_check(B, T, H, K, V, L);
    if (rc != 0) return rc;
    if (!q || !k || !v || !beta || !g_cum || !lambda || !Aw || !Au || !d_o || !d_qd || !d_wd || !d_kd || !d_u || !d_gl || !dlambda)
        return LLATTN_ERR_NULL;
    llattn::GdnParams p = {};
    p.B = B; p.T = T; p.H = H; p.K = K; p.V = V; p.L = L;
    const size_t need = gdn_setup(p, nullptr, GDN_WS_CHUNK | GDN_WS_HS | GDN_WS_DHS);
    if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255)) return LLATTN_ERR_WORKSPACE;
    gdn_setup(p, workspace, GDN_WS_CHUNK | GDN_WS_HS | GDN_WS_DHS);
    p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v;
    p.beta = (const __nv_bfloat16*)beta; p.g = nullptr; p.l = (const __nv_bfloat16*)lambda;
    p.g_cum = const_cast<float*>(g_cum);
    p.Aw = (__nv_bfloat16*)const_cast<void*>(Aw); p.Au = (__nv_bfloat16*)const_cast<void*>(Au);
    p.d_o = (const __nv_bfloat16*)d_o;
    p.d_qd = d_qd; p.d_wd = d_wd; p.d_kd = d_kd; p.d_u = (__nv_bfloat16*)d_u; p.d_gl = d_gl; p.dl = dlambda;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e0 = cudaMemsetAsync(p.err, 0, sizeof(int), st);
    if (e0 != cudaSuccess) return (int)e0;
    if ((rc = llattn::gdn_recompute_dispatch(p, st)) != 0) return rc;
    if ((rc = llattn::gdn_bwd_scan_dispatch(p, st)) != 0) return rc;
    return llattn::gdn_bwd_levels_dispatch(p, st);
}

static size_t gdn_bwd_setup(llattn::GdnParams& p, void* ws, bool kept = false) {
    // with the forward call's workspace kept, only the adjoint states and the intermediate gradients are needed
    const size_t base = gdn_setup(p, ws, kept ? GDN_WS_DHS : (GDN_WS_CHUNK | GDN_WS_HS | GDN_WS_DHS));
    Carver c(ws);
    c.off = base;
    const size_t n = (size_t)p.B * p.T * p.H;
    p.d_qd = c.take<float>(n * p.K);
    p.d_wd = c.take<float>(n * p.K);
    p.d_kd = c.take<float>(n * p.K);
    p.d_u = c.take<__nv_bfloat16>(n * p.V);
    p.d_gl = c.take<float>((size_t)p.B * p.NT * p.H);
    p.dqd_neg = c.take<__nv_bfloat16>(n * p.K);
    p.d_grow = c.take<float>(n);
    return c.off;
}

size_t llattn_gdn_bwd_workspace_bytes(int B, int T, int H, int K, int V, int L) {
    if (gdn_check(B, T, H, K, V, L) != 0) return 0;
    llattn::GdnParams p = {};
    p.B = B; p.T = T; p.H = H; p.K = K; p.V = V; p.L = L;
    return gdn_bwd_setup(p, nullptr);
}

static int gdn_bwd_impl(const void* q, const void* k, const void* v, const void* beta, const float* g_cum, const void* lambda,
                        const void* Aw, const void* Au, const void* d_o, float* dq, float* dk, float* dv, float* dbeta, float* dg,
                        float* dlambda, const void* fwd_workspace, size_t fwd_workspace_bytes, void* workspace,
                        size_t workspace_bytes, int B, int T, int H, int K, int V, int L, void* stream, void* dv_bf16 = nullptr) {
    int rc = gdn_check(B, T, H, K, V, L);
    if (rc != 0) return rc;
    if (!q || !k || !v || !beta || !g_cum || !lambda || !Aw || !Au || !d_o || !dq || !dk || (!dv && !dv_bf16) || !dbeta || !dg || !dlambda)
        return LLATTN_ERR_NULL;
    llattn::GdnParams p = {};
    p.B = B; p.T = T; p.H = H; p.K = K; p.V = V; p.L = L;
    const bool kept = fwd_workspace != nullptr;
    if (kept) {
        // chunk matrices and level states as llattn_gdn_fwd_keep left them
        const size_t fneed = gdn_setup(p, nullptr, GDN_WS_CHUNK | GDN_WS_HS);
        if (fwd_workspace_bytes < fneed || ((uintptr_t)fwd_workspace & 255)) return LLATTN_ERR_WORKSPACE;
        gdn_setup(p, const_cast<void*>(fwd_workspace), GDN_WS_CHUNK | GDN_WS_HS);
    }
    const size_t need = gdn_bwd_setup(p, nullptr, kept);
    if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255)) return LLATTN_ERR_WORKSPACE;
    gdn_bwd_setup(p, workspace, kept);
    p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v;
    p.beta = (const __nv_bfloat16*)beta; p.g = nullptr; p.l = (const __nv_bfloat16*)lambda;
    p.g_cum = const_cast<float*>(g_cum);
    p.Aw = (__nv_bfloat16*)const_cast<void*>(Aw); p.Au = (__nv_bfloat16*)const_cast<void*>(Au);
    p.d_o = (const __nv_bfloat16*)d_o;
    p.dq = dq; p.dk = dk; p.dv = dv; p.dv_bf16 = (__nv_bfloat16*)dv_bf16; p.dbeta = dbeta; p.dg = dg; p.dl = dlambda;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(dlambda, 0, (size_t)B * T * H * L * sizeof(float), st);
    if (e != cudaSuccess) return (int)e;
    if ((e = cudaMemsetAsync(p.err, 0, sizeof(int), st)) != cudaSuccess) return (int)e;
    if (!kept && (rc = llattn::gdn_recompute_dispatch(p, st)) != 0) return rc;
    if ((rc = llattn::gdn_bwd_scan_dispatch(p, st)) != 0) return rc;
    if (!llattn::gdn_bwd_levels_writes_row_terms(p)) {
        p.dqd_neg = nullptr;
        p.d_grow = nullptr;
    }
    if ((rc = llattn::gdn_bwd_levels_dispatch(p, st)) != 0) return rc;
    return llattn::gdn_bwd_chunk_dispatch(p, st);
}

int llattn_gdn_bwd(const void* q, const void* k, const void* v, const void* beta, const float* g_cum, const void* lambda,
                   const void* Aw, const void* Au, const void* d_o, float* dq, float* dk, float* dv, float* dbeta, float* dg,
                   float* dlambda, void* workspace, size_t workspace_bytes,
                   int B, int T, int H, int K, int V, int L, void* stream) {
    return gdn_bwd_impl(q, k, v, beta, g_cum, lambda, Aw, Au, d_o, dq, dk, dv, dbeta, dg, dlambda, nullptr, 0, workspace,
                        workspace_bytes, B, T, H, K, V, L, stream);
}

int llattn_gdn_bwd_kept_bf16dv(const void* q, const void* k, const void* v, const void* beta, const float* g_cum, const void* lambda,
                               const void* Aw, const void* Au, const void* d_o, float* dq, float* dk, void* dv_bf16, float* dbeta,
                               float* dg, float* dlambda, const void* fwd_workspace, size_t fwd_workspace_bytes, void* workspace,
                               size_t workspace_bytes, int B, int T, int H, int K, int V, int L, void* stream) {
    if (!fwd_workspace || !dv_bf16) return LLATTN_ERR_NULL;
    return gdn_bwd_impl(q, k, v, beta, g_cum, lambda, Aw, Au, d_o, dq, dk, nullptr, dbeta, dg, dlambda, fwd_workspace,
                        fwd_workspace_bytes, workspace, workspace_bytes, B, T, H, K, V, L, stream, dv_bf16);
}

size_t llattn_gdn_bwd_kept_workspace_bytes(int B, int T, int H, int K, int V, int L) {
    if (gdn_check(B, T, H, K, V, L) != 0) return 0;
    llattn::GdnParams p = {};
    p.B = B; p.T = T; p.H = H; p.K = K; p.V = V; p.L = L;
    return gdn_bwd_setup(p, nullptr, true);
}

int llattn_gdn_bwd_kept(const void* q, const void* k, const void* v, const void* beta, const float* g_cum, const void* lambda,
                        const void* Aw, const void* Au, const void* d_o, float* dq, float* dk, float* dv, float* dbeta,
                        float* dg, float* dlambda, const void* fwd_workspace, size_t fwd_workspace_bytes, void* workspace,
                        size_t workspace_bytes, int B, int T, int H, int K, int V, int L, void* stream) {
    if (!fwd_workspace) return LLATTN_ERR_NULL;
    return gdn_bwd_impl(q, k, v, beta, g_cum, lambda, Aw, Au, d_o, dq, dk, dv, dbeta, dg, dlambda, fwd_workspace,
                        fwd_workspace_bytes, workspace, workspace_bytes, B, T, H, K, V, L, stream);
}

}  // extern "C"
