// Grouped and spatial shapes: repack -> 2-D kernels per group -> scatter back.
//
// A general call has x [B, G, CIg, HW].  Every (b, hw) pair is one sample of group g's 2-D
// problem, and all HW samples of a row share the row's 32-row sub-batch (= its mask lists).  The
// packed copy orders the samples so that the 2-D kernels' own rule "sub-batch = row / 32" stays
// true: packed row r = ((b / 32) * HW + hw) * 32 + b % 32, i.e. packed sub-batch s' = s * HW + hw,
// and the mask lists are replicated to [S * HW] rows accordingly.  A last, partial sub-batch is
// padded to 32 rows with zeros (ones for the saved l-p outputs, whose reciprocal is taken), and the
// padding rows' results are dropped on the way back.  Group g of the packed operands is a
// contiguous row-major [B', C] matrix, group g of w is the contiguous slab of rows
// g*W_COg .. (g+1)*W_COg - 1, so the 2-D entry points run on them unchanged.
//
// The repacking moves O(B * HW * (CI + CO)) words next to O(B * HW * CI * CO / G) arithmetic, so
// plain one-word-per-thread kernels are enough.  Scratch comes from the stream-ordered allocator
// (a pool of this library's own, cudaMallocFromPoolAsync / cudaFreeAsync on the caller's stream);
// the 2-D fast path never gets here.
#include "general_shapes.h"

#include "../../include/sortnet_b200.h"
#include "common.cuh"
#include "launch.h"

namespace snb {
namespace {

struct Geo {
    int B, G, HW, S, Bp;  // Bp = S * HW * 32 packed rows per group
};

// src [K][B][G][C][HW] -> dst [G][K][Bp][C]; padding rows get `fill`.
__global__ void pack_rows_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, Geo q, int C,
                                 int K, uint32_t fill, long long n) {
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < n;
         idx += (long long)gridDim.x * blockDim.x) {
        int c = (int)(idx % C);
        long long t = idx / C;
        int r = (int)(t % q.Bp);
        t /= q.Bp;
        int k = (int)(t % K), g = (int)(t / K);
        int sh = r >> 5, hw = sh % q.HW, b = (sh / q.HW) * 32 + (r & 31);
        dst[idx] = b < q.B ? src[((((long long)k * q.B + b) * q.G + g) * C + c) * q.HW + hw] : fill;
    }
}

// src [G][K][Bp][C] -> dst [K][B][G][C][HW].
__global__ void unpack_rows_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, Geo q, int C,
                                   int K, long long n) {
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < n;
         idx += (long long)gridDim.x * blockDim.x) {
        int hw = (int)(idx % q.HW);
        long long t = idx / q.HW;
        int c = (int)(t % C);
        t /= C;
        int g = (int)(t % q.G);
        t /= q.G;
        int b = (int)(t % q.B), k = (int)(t / q.B);
        int r = ((b >> 5) * q.HW + hw) * 32 + (b & 31);
        dst[idx] = src[(((long long)g * K + k) * q.Bp + r) * C + c];
    }
}

// m [S][G][C] -> mp [G][S][HW][C]: every spatial position of a sub-batch uses the same list.
__global__ void expand_mask_kernel(const int* __restrict__ m, int* __restrict__ mp, Geo q, int C, long long n) {
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < n;
         idx += (long long)gridDim.x * blockDim.x) {
        int c = (int)(idx % C);
        long long t = idx / C / q.HW;
        int s = (int)(t % q.S), g = (int)(t / q.S);
        mp[idx] = m[((long long)s * q.G + g) * C + c];
    }
}

inline int grid_for(long long n) { return (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16); }

// The library's own memory pools, one per device, created on first use (see Arena::commit).
// Freed scratch up to SCRATCH_KEEP_BYTES stays in a pool between calls; snb_trim_scratch() hands
// it back to the driver.
constexpr unsigned long long SCRATCH_KEEP_BYTES = 2ull << 30;
inline std::mutex& pool_mutex() {
    static std::mutex m;
    return m;
}
inline cudaMemPool_t* pool_table() {
    static cudaMemPool_t pools[64] = {};
    return pools;
}

// One stream-ordered allocation carved into 256-byte aligned pieces.
class Arena {
  public:
    explicit Arena(cudaStream_t st) : st_(st) {}
    ~Arena() {
        if (base_) cudaFreeAsync(base_, st_);
    }
    size_t reserve(size_t bytes) {
        size_t o = total_;
        total_ += (bytes + 255) & ~(size_t)255;
        return o;
    }
    cudaError_t commit() {
        // A memory pool of this library's own per device, with the release threshold raised so that
        // freed scratch (up to 2 GiB) stays in the pool and the next call reuses it (a pool with the
        // default threshold of 0 hands its memory back to the driver at the next synchronisation,
        // which made every call pay for fresh physical memory).  The device's default pool is left
        // alone.  The table is guarded: two host threads may make their first call at once.
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
        std::lock_guard<std::mutex> lock(pool_mutex());
        cudaMemPool_t* pools = pool_table();
        if (!pools[dev]) {
            cudaMemPoolProps props = {};
            props.allocType = cudaMemAllocationTypePinned;
            props.handleTypes = cudaMemHandleTypeNone;
            props.location.type = cudaMemLocationTypeDevice;
            props.location.id = dev;
            cudaMemPool_t pool;
            e = cudaMemPoolCreate(&pool, &props);
            if (e != cudaSuccess) return e;
            unsigned long long keep = SCRATCH_KEEP_BYTES;
            e = cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
            if (e != cudaSuccess) return e;
            pools[dev] = pool;
        }
        return cudaMallocFromPoolAsync((void**)&base_, total_ ? total_ : 256, pools[dev], st_);
    }
    template <class T>
    T* at(size_t off) const { return reinterpret_cast<T*>(base_ + off); }

  private:
    cudaStream_t st_;
    char* base_ = nullptr;
    size_t total_ = 0;
};

int make_geo(int B, int CO, int CI, int G, int HW, int W_CO, Geo* q) {
    if (G < 1 || HW < 1 || B <= 0 || CO <= 0 || CI <= 0) return SNB_ERR_BAD_SHAPE;
    if (CO % G || CI % G || (W_CO > 0 && W_CO % G)) return SNB_ERR_BAD_SHAPE;
    long long S = (B + 31) / 32, Bp = S * HW * 32;
    if (Bp >= (1ll << 31) || Bp * (CI / G) >= (1ll << 31) || Bp * (CO / G) >= (1ll << 31)) return SNB_ERR_TOO_LARGE;
    *q = Geo{B, G, HW, (int)S, (int)Bp};
    return SNB_OK;
}

size_t words(const Geo& q, int C, int K = 1) { return sizeof(uint32_t) * (size_t)q.G * K * q.Bp * C; }

cudaError_t pack(const void* src, void* dst, const Geo& q, int C, int K, uint32_t fill, cudaStream_t st) {
    long long n = (long long)q.G * K * q.Bp * C;
    pack_rows_kernel<<<grid_for(n), 256, 0, st>>>((const uint32_t*)src, (uint32_t*)dst, q, C, K, fill, n);
    return cudaGetLastError();
}
cudaError_t unpack(const void* src, void* dst, const Geo& q, int C, int K, cudaStream_t st) {
    long long n = (long long)K * q.B * q.G * C * q.HW;
    unpack_rows_kernel<<<grid_for(n), 256, 0, st>>>((const uint32_t*)src, (uint32_t*)dst, q, C, K, n);
    return cudaGetLastError();
}
cudaError_t expand(const int* m, int* mp, const Geo& q, int C, cudaStream_t st) {
    long long n = (long long)q.G * q.S * q.HW * C;
    expand_mask_kernel<<<grid_for(n), 256, 0, st>>>(m, mp, q, C, n);
    return cudaGetLastError();
}
size_t mask_bytes(const Geo& q, int C) { return sizeof(int) * (size_t)q.G * q.S * q.HW * C; }
// Group g of a packed matrix / an expanded mask / the weights.
template <class T>
T* grp(T* base, const Geo& q, int g, int C, int K = 1) { return base + (size_t)g * K * q.Bp * C; }
const int* mgrp(const int* base, const Geo& q, int g, int C) {
    return base ? base + (size_t)g * q.S * q.HW * C : nullptr;
}

constexpr uint32_t ONE_BITS = 0x3f800000u;  // 1.0f

}  // namespace

int general_inf_forward(const float* x, const float* w, int B, int CO, int CI, int G, int HW, float* y,
                        int* pos, const int* ci, const int* co, int W_CO, int W_CI, cudaStream_t st) {
    if (!x || !w || !y) return SNB_ERR_NULL_POINTER;
    Geo q;
    if (int rc = make_geo(B, CO, CI, G, HW, W_CO, &q)) return rc;
    if ((pos == nullptr) && (ci || co)) return SNB_ERR_UNSUPPORTED;
    if (W_CI <= 0 || W_CI % G) return SNB_ERR_BAD_SHAPE;
    const int COg = CO / G, CIg = CI / G, W_COg = W_CO / G, W_CIg = W_CI / G;
    Arena a(st);
    size_t ox = a.reserve(words(q, CIg)), oy = a.reserve(words(q, COg));
    size_t op = pos ? a.reserve(words(q, COg)) : 0;
    size_t oci = ci ? a.reserve(mask_bytes(q, CIg)) : 0, oco = co ? a.reserve(mask_bytes(q, COg)) : 0;
    size_t ws_bytes = pos ? snb_inf_dist_forward_workspace_bytes(q.Bp, COg) : 0;
    size_t ows = a.reserve(ws_bytes);
    SNB_CUDA(a.commit());
    float *xp = a.at<float>(ox), *yp = a.at<float>(oy);
    int* pp = pos ? a.at<int>(op) : nullptr;
    int *cip = ci ? a.at<int>(oci) : nullptr, *cop = co ? a.at<int>(oco) : nullptr;
    SNB_CUDA(pack(x, xp, q, CIg, 1, 0u, st));
    if (ci) SNB_CUDA(expand(ci, cip, q, CIg, st));
    if (co) SNB_CUDA(expand(co, cop, q, COg, st));
    for (int g = 0; g < G; g++) {
        const float* wg = w + (size_t)g * W_COg * W_CIg;
        int rc = pos ? snb_inf_dist_forward_ws(grp(xp, q, g, CIg), wg, q.Bp, COg, CIg, 1, 1, grp(yp, q, g, COg),
                                               grp(pp, q, g, COg), mgrp(cip, q, g, CIg), mgrp(cop, q, g, COg),
                                               W_COg, W_CIg, a.at<void>(ows), ws_bytes, st)
                     : snb_inf_dist_forward_nograd(grp(xp, q, g, CIg), wg, q.Bp, COg, CIg, 1, 1,
                                                   grp(yp, q, g, COg), st);
        if (rc) return rc;
    }
    SNB_CUDA(unpack(yp, y, q, COg, 1, st));
    if (pos) SNB_CUDA(unpack(pp, pos, q, COg, 1, st));
    return SNB_OK;
}

int general_inf_backward(const float* g_, const int* pos, int B, int CO, int CI, int G, int HW, float* gx,
                         float* gw, const int* ci, const int* co, int W_CO, int W_CI, cudaStream_t st) {
    if (!g_ || !pos || !gx) return SNB_ERR_NULL_POINTER;
    Geo q;
    if (int rc = make_geo(B, CO, CI, G, HW, gw ? W_CO : 0, &q)) return rc;
    if (W_CI <= 0 || W_CI % G) return SNB_ERR_BAD_SHAPE;
    const int COg = CO / G, CIg = CI / G, W_COg = W_CO / G, W_CIg = W_CI / G;
    Arena a(st);
    size_t og = a.reserve(words(q, COg)), op = a.reserve(words(q, COg)), ox = a.reserve(words(q, CIg));
    size_t oci = (gw && ci) ? a.reserve(mask_bytes(q, CIg)) : 0, oco = (gw && co) ? a.reserve(mask_bytes(q, COg)) : 0;
    SNB_CUDA(a.commit());
    float *gp = a.at<float>(og), *gxp = a.at<float>(ox);
    int* pp = a.at<int>(op);
    int *cip = (gw && ci) ? a.at<int>(oci) : nullptr, *cop = (gw && co) ? a.at<int>(oco) : nullptr;
    SNB_CUDA(pack(g_, gp, q, COg, 1, 0u, st));
    SNB_CUDA(pack(pos, pp, q, COg, 1, 0u, st));
    if (cip) SNB_CUDA(expand(ci, cip, q, CIg, st));
    if (cop) SNB_CUDA(expand(co, cop, q, COg, st));
    for (int g = 0; g < G; g++) {
        int rc = gw ? snb_inf_dist_backward_input_weight(grp(gp, q, g, COg), grp(pp, q, g, COg), q.Bp, COg, CIg, 1, 1,
                                                         grp(gxp, q, g, CIg), gw + (size_t)g * W_COg * W_CIg,
                                                         mgrp(cip, q, g, CIg), mgrp(cop, q, g, COg), W_COg, W_CIg, st)
                    : snb_inf_dist_backward_input(grp(gp, q, g, COg), grp(pp, q, g, COg), q.Bp, COg, CIg, 1, 1,
                                                  grp(gxp, q, g, CIg), st);
        if (rc) return rc;
    }
    SNB_CUDA(unpack(gxp, gx, q, CIg, 1, st));
    return SNB_OK;
}

int general_lp_forward(const float* x, const float* w, int B, int CO, int CI, int G, int HW, float* y,
                       float p, const int* ci, const int* co, int W_CO, int W_CI, cudaStream_t st) {
    if (!x || !w || !y) return SNB_ERR_NULL_POINTER;
    Geo q;
    if (int rc = make_geo(B, CO, CI, G, HW, W_CO, &q)) return rc;
    if (W_CI <= 0 || W_CI % G) return SNB_ERR_BAD_SHAPE;
    const int COg = CO / G, CIg = CI / G, W_COg = W_CO / G, W_CIg = W_CI / G;
    Arena a(st);
    size_t ox = a.reserve(words(q, CIg)), oy = a.reserve(words(q, COg));
    size_t oci = ci ? a.reserve(mask_bytes(q, CIg)) : 0, oco = co ? a.reserve(mask_bytes(q, COg)) : 0;
    const size_t ws_bytes = snb_norm_dist_forward_workspace_bytes(q.Bp, COg, p);
    size_t ows = a.reserve(ws_bytes);
    SNB_CUDA(a.commit());
    float *xp = a.at<float>(ox), *yp = a.at<float>(oy);
    int *cip = ci ? a.at<int>(oci) : nullptr, *cop = co ? a.at<int>(oco) : nullptr;
    SNB_CUDA(pack(x, xp, q, CIg, 1, 0u, st));
    if (ci) SNB_CUDA(expand(ci, cip, q, CIg, st));
    if (co) SNB_CUDA(expand(co, cop, q, COg, st));
    for (int g = 0; g < G; g++) {
        int rc = snb_norm_dist_forward_ws(grp(xp, q, g, CIg), w + (size_t)g * W_COg * W_CIg, q.Bp, COg, CIg, 1, 1,
                                          grp(yp, q, g, COg), p, mgrp(cip, q, g, CIg), mgrp(cop, q, g, COg), W_COg,
                                          W_CIg, ws_bytes ? a.at<void>(ows) : nullptr, ws_bytes, st);
        if (rc) return rc;
    }
    SNB_CUDA(unpack(yp, y, q, COg, 1, st));
    return SNB_OK;
}

int general_lp_backward(const float* g_, const float* x, const float* w, const float* y, int B, int CO,
                        int CI, int G, int HW, float* gx, float* gw, float p, const int* ci,
                        const int* co, int W_CO, int W_CI, cudaStream_t st) {
    if (!g_ || !x || !w || !y || !gx) return SNB_ERR_NULL_POINTER;
    Geo q;
    if (int rc = make_geo(B, CO, CI, G, HW, W_CO, &q)) return rc;
    if (W_CI <= 0 || W_CI % G) return SNB_ERR_BAD_SHAPE;
    const int COg = CO / G, CIg = CI / G, W_COg = W_CO / G, W_CIg = W_CI / G;
    Arena a(st);
    size_t og = a.reserve(words(q, COg)), oy = a.reserve(words(q, COg));
    size_t ox = a.reserve(words(q, CIg)), ogx = a.reserve(words(q, CIg));
    size_t oci = ci ? a.reserve(mask_bytes(q, CIg)) : 0, oco = co ? a.reserve(mask_bytes(q, COg)) : 0;
    SNB_CUDA(a.commit());
    float *gp = a.at<float>(og), *yp = a.at<float>(oy), *xp = a.at<float>(ox), *gxp = a.at<float>(ogx);
    int *cip = ci ? a.at<int>(oci) : nullptr, *cop = co ? a.at<int>(oco) : nullptr;
    SNB_CUDA(pack(g_, gp, q, COg, 1, 0u, st));
    SNB_CUDA(pack(y, yp, q, COg, 1, ONE_BITS, st));  // padding rows: gradient 0 over output 1
    SNB_CUDA(pack(x, xp, q, CIg, 1, 0u, st));
    if (ci) SNB_CUDA(expand(ci, cip, q, CIg, st));
    if (co) SNB_CUDA(expand(co, cop, q, COg, st));
    for (int g = 0; g < G; g++) {
        const float* wg = w + (size_t)g * W_COg * W_CIg;
        int rc = gw ? snb_norm_dist_backward_input_weight(grp(gp, q, g, COg), grp(xp, q, g, CIg), wg,
                                                          grp(yp, q, g, COg), q.Bp, COg, CIg, 1, 1,
                                                          grp(gxp, q, g, CIg), gw + (size_t)g * W_COg * W_CIg, p,
                                                          mgrp(cip, q, g, CIg), mgrp(cop, q, g, COg), W_COg, W_CIg, st)
                    : snb_norm_dist_backward_input(grp(gp, q, g, COg), grp(xp, q, g, CIg), wg, grp(yp, q, g, COg),
                                                   q.Bp, COg, CIg, 1, 1, grp(gxp, q, g, CIg), p,
                                                   mgrp(cip, q, g, CIg), mgrp(cop, q, g, COg), W_COg, W_CIg, st);
        if (rc) return rc;
    }
    SNB_CUDA(unpack(gxp, gx, q, CIg, 1, st));
    return SNB_OK;
}

int general_bound_forward(const float* xl, const float* xu, const float* w, int B, int CO, int CI, int G,
                          int HW, float* yl, float* yu, int* posl, int* posu, cudaStream_t st) {
    if (!xl || !xu || !w || !yl || !yu) return SNB_ERR_NULL_POINTER;
    if ((posl == nullptr) != (posu == nullptr)) return SNB_ERR_NULL_POINTER;
    Geo q;
    if (int rc = make_geo(B, CO, CI, G, HW, CO, &q)) return rc;
    const int COg = CO / G, CIg = CI / G;
    Arena a(st);
    size_t oxl = a.reserve(words(q, CIg)), oxu = a.reserve(words(q, CIg));
    size_t oyl = a.reserve(words(q, COg)), oyu = a.reserve(words(q, COg));
    size_t opl = posl ? a.reserve(words(q, COg)) : 0, opu = posl ? a.reserve(words(q, COg)) : 0;
    SNB_CUDA(a.commit());
    float *xlp = a.at<float>(oxl), *xup = a.at<float>(oxu), *ylp = a.at<float>(oyl), *yup = a.at<float>(oyu);
    int *plp = posl ? a.at<int>(opl) : nullptr, *pup = posl ? a.at<int>(opu) : nullptr;
    SNB_CUDA(pack(xl, xlp, q, CIg, 1, 0u, st));
    SNB_CUDA(pack(xu, xup, q, CIg, 1, 0u, st));
    for (int g = 0; g < G; g++) {
        const float* wg = w + (size_t)g * COg * CIg;
        int rc = posl ? snb_bound_inf_dist_forward(grp(xlp, q, g, CIg), grp(xup, q, g, CIg), wg, q.Bp, COg, CIg, 1, 1,
                                                   grp(ylp, q, g, COg), grp(yup, q, g, COg), grp(plp, q, g, COg),
                                                   grp(pup, q, g, COg), st)
                      : snb_bound_inf_dist_forward_nograd(grp(xlp, q, g, CIg), grp(xup, q, g, CIg), wg, q.Bp, COg,
                                                          CIg, 1, 1, grp(ylp, q, g, COg), grp(yup, q, g, COg), st);
        if (rc) return rc;
    }
    SNB_CUDA(unpack(ylp, yl, q, COg, 1, st));
    SNB_CUDA(unpack(yup, yu, q, COg, 1, st));
    if (posl) {
        SNB_CUDA(unpack(plp, posl, q, COg, 1, st));
        SNB_CUDA(unpack(pup, posu, q, COg, 1, st));
    }
    return SNB_OK;
}

int general_bound_backward(const float* gl, const float* gu, const int* posl, const int* posu, int B,
                           int CO, int CI, int G, int HW, float* gxl, float* gxu, float* gw,
                           cudaStream_t st) {
    if (!gl || !gu || !posl || !posu || !gxl || !gxu) return SNB_ERR_NULL_POINTER;
    Geo q;
    if (int rc = make_geo(B, CO, CI, G, HW, CO, &q)) return rc;
    const int COg = CO / G, CIg = CI / G;
    Arena a(st);
    size_t ogl = a.reserve(words(q, COg)), ogu = a.reserve(words(q, COg));
    size_t opl = a.reserve(words(q, COg)), opu = a.reserve(words(q, COg));
    size_t oxl = a.reserve(words(q, CIg)), oxu = a.reserve(words(q, CIg));
    SNB_CUDA(a.commit());
    float *glp = a.at<float>(ogl), *gup = a.at<float>(ogu), *gxlp = a.at<float>(oxl), *gxup = a.at<float>(oxu);
    int *plp = a.at<int>(opl), *pup = a.at<int>(opu);
    SNB_CUDA(pack(gl, glp, q, COg, 1, 0u, st));
    SNB_CUDA(pack(gu, gup, q, COg, 1, 0u, st));
    SNB_CUDA(pack(posl, plp, q, COg, 1, SNB_NO_GRAD_ID, st));  // padding rows: "no gradient" word
    SNB_CUDA(pack(posu, pup, q, COg, 1, 0u, st));
    for (int g = 0; g < G; g++) {
        int rc = gw ? snb_bound_inf_dist_backward_input_weight(
                          grp(glp, q, g, COg), grp(gup, q, g, COg), grp(plp, q, g, COg), grp(pup, q, g, COg), q.Bp,
                          COg, CIg, 1, 1, grp(gxlp, q, g, CIg), grp(gxup, q, g, CIg), gw + (size_t)g * COg * CIg, st)
                    : snb_bound_inf_dist_backward_input(grp(glp, q, g, COg), grp(gup, q, g, COg), grp(plp, q, g, COg),
                                                        grp(pup, q, g, COg), q.Bp, COg, CIg, 1, 1,
                                                        grp(gxlp, q, g, CIg), grp(gxup, q, g, CIg), st);
        if (rc) return rc;
    }
    SNB_CUDA(unpack(gxlp, gxl, q, CIg, 1, st));
    SNB_CUDA(unpack(gxup, gxu, q, CIg, 1, st));
    return SNB_OK;
}

int general_sort_forward(const float* x, const float* w, int B, int CO, int CI, int G, int HW, float* y,
                         int* pos, float qq, int K, cudaStream_t st) {
    if (!x || !w || !y) return SNB_ERR_NULL_POINTER;
    if (K < 2 || K > 25) return SNB_ERR_UNSUPPORTED;
    Geo q;
    if (int rc = make_geo(B, CO, CI, G, HW, CO, &q)) return rc;
    const int COg = CO / G, CIg = CI / G;
    Arena a(st);
    size_t ox = a.reserve(words(q, CIg)), oy = a.reserve(words(q, COg));
    size_t op = pos ? a.reserve(words(q, COg, K)) : 0;
    SNB_CUDA(a.commit());
    float *xp = a.at<float>(ox), *yp = a.at<float>(oy);
    int* pp = pos ? a.at<int>(op) : nullptr;
    SNB_CUDA(pack(x, xp, q, CIg, 1, 0u, st));
    for (int g = 0; g < G; g++) {
        const float* wg = w + (size_t)g * COg * CIg;
        int rc = pos ? snb_sort_neuron_forward(grp(xp, q, g, CIg), wg, q.Bp, COg, CIg, 1, 1, grp(yp, q, g, COg),
                                               grp(pp, q, g, COg, K), qq, K, st)
                     : snb_sort_neuron_forward_nograd(grp(xp, q, g, CIg), wg, q.Bp, COg, CIg, 1, 1,
                                                      grp(yp, q, g, COg), qq, K, st);
        if (rc) return rc;
    }
    SNB_CUDA(unpack(yp, y, q, COg, 1, st));
    if (pos) SNB_CUDA(unpack(pp, pos, q, COg, K, st));
    return SNB_OK;
}

int general_sort_bound_forward(const float* xl, const float* xu, const float* w, int B, int CO, int CI,
                               int G, int HW, float* yl, float* yu, float qq, int K, cudaStream_t st) {
    if (!xl || !xu || !w || !yl || !yu) return SNB_ERR_NULL_POINTER;
    Geo q;
    if (int rc = make_geo(B, CO, CI, G, HW, CO, &q)) return rc;
    const int COg = CO / G, CIg = CI / G;
    Arena a(st);
    size_t oxl = a.reserve(words(q, CIg)), oxu = a.reserve(words(q, CIg));
    size_t oyl = a.reserve(words(q, COg)), oyu = a.reserve(words(q, COg));
    SNB_CUDA(a.commit());
    float *xlp = a.at<float>(oxl), *xup = a.at<float>(oxu), *ylp = a.at<float>(oyl), *yup = a.at<float>(oyu);
    SNB_CUDA(pack(xl, xlp, q, CIg, 1, 0u, st));
    SNB_CUDA(pack(xu, xup, q, CIg, 1, 0u, st));
    for (int g = 0; g < G; g++) {
        int rc = snb_bound_sort_neuron_forward(grp(xlp, q, g, CIg), grp(xup, q, g, CIg), w + (size_t)g * COg * CIg,
                                               q.Bp, COg, CIg, 1, 1, grp(ylp, q, g, COg), grp(yup, q, g, COg), qq, K,
                                               st);
        if (rc) return rc;
    }
    SNB_CUDA(unpack(ylp, yl, q, COg, 1, st));
    SNB_CUDA(unpack(yup, yu, q, COg, 1, st));
    return SNB_OK;
}

int general_sort_backward(const float* g_, const int* pos, int B, int CO, int CI, int G, int HW, float* gx,
                          float* gw, float qq, int K, cudaStream_t st) {
    if (!g_ || !pos || !gx) return SNB_ERR_NULL_POINTER;
    if (K < 2 || K > 25) return SNB_ERR_UNSUPPORTED;
    Geo q;
    if (int rc = make_geo(B, CO, CI, G, HW, CO, &q)) return rc;
    const int COg = CO / G, CIg = CI / G;
    Arena a(st);
    size_t og = a.reserve(words(q, COg)), op = a.reserve(words(q, COg, K)), ox = a.reserve(words(q, CIg));
    SNB_CUDA(a.commit());
    float *gp = a.at<float>(og), *gxp = a.at<float>(ox);
    int* pp = a.at<int>(op);
    SNB_CUDA(pack(g_, gp, q, COg, 1, 0u, st));
    SNB_CUDA(pack(pos, pp, q, COg, K, 0u, st));
    for (int g = 0; g < G; g++) {
        int rc = gw ? snb_sort_neuron_backward_input_weight(grp(gp, q, g, COg), grp(pp, q, g, COg, K), q.Bp, COg, CIg,
                                                            1, 1, grp(gxp, q, g, CIg), gw + (size_t)g * COg * CIg, qq,
                                                            K, st)
                    : snb_sort_neuron_backward_input(grp(gp, q, g, COg), grp(pp, q, g, COg, K), q.Bp, COg, CIg, 1, 1,
                                                     grp(gxp, q, g, CIg), qq, K, st);
        if (rc) return rc;
    }
    SNB_CUDA(unpack(gxp, gx, q, CIg, 1, st));
    return SNB_OK;
}

}  // namespace snb

// Returns the scratch that the grouped / spatial shapes left in this library's memory pool of the
// current device to the driver (the pool keeps up to 2 GiB of freed scratch for reuse otherwise).
// Synchronises nothing; memory still in use by queued work stays until that work has finished.
extern "C" int snb_trim_scratch(void) {
    int dev = 0;
    SNB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return SNB_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(snb::pool_mutex());
    cudaMemPool_t pool = snb::pool_table()[dev];
    if (pool) SNB_CUDA(cudaMemPoolTrimTo(pool, 0));
    return SNB_OK;
}
