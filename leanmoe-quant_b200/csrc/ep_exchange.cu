// Row bookkeeping of the expert-parallel exchange (batched decode over several GPUs): everything between the
// routing and the all-to-all, and between the all-to-all and the expert kernels, as a handful of kernels instead of
// some forty library launches (sort, gather, scatter, cumulative sums, fills) per layer.
//
// A rank holds T tokens with K routed experts each: P = T * K pairs.  Expert e lives on rank e / epr.  The send
// buffer has `world` blocks of P row slots (the static capacity: the worst case for every peer), a row is the token's
// H activations followed by 8 more fp16 values of which the first is the expert id; unused slots carry the id
// `experts`.  Pairs are placed in the order "expert id, then pair index" (a stable sort), so every rank can undo the
// order without exchanging anything but the rows.  The receiver regroups its world * P slots by local expert (stable
// again), which also yields the segment offsets the grouped expert kernels want.
//
//   dispatch : plan (one block: counting sort of the pairs)        + rows into the send slots (one block per slot)
//   regroup  : plan (one block: counting sort of the received ids) + rows into expert order   (one block per row)
//   give back: results from expert order to the slots they came in (one block per row)
//   combine  : out[t] = sum_k w[t, k] * back[slot(t, k)] in slot order, fp32                  (one block per token)
//
// Index work on a few hundred pairs: one block per plan is enough; a pair's place among its equals is found by
// counting the equal ids before it (P <= 4096).  No atomics on data, the order is fixed.
#include "common.cuh"
#include "kernels.h"

namespace lemoq {
namespace {

constexpr int kIdCols = 8;        // fp16 values behind the activations of a row; [0] is the expert id
constexpr int kPlanThreads = 512;
constexpr int kMaxPlanItems = 4096;
constexpr int kMaxPlanKeys = 2048;

// Stable counting sort of n keys in [0, nkeys) held in shared memory: rank_of[i] = place of item i.  first[k] = place of
// the first item with key k (first[nkeys] = n).  Called by the whole block.
__device__ void stable_places(const int* keys, int n, int nkeys, int* first, int* place) {
    for (int k = threadIdx.x; k <= nkeys; k += blockDim.x) first[k] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&first[keys[i] + 1], 1);  // counts only: order-free
    __syncthreads();
    if (threadIdx.x < 32) {  // inclusive scan of the counts by one warp, 32 keys at a time
        int carry = 0;
        for (int k0 = 1; k0 <= nkeys; k0 += 32) {
            const int k = k0 + static_cast<int>(threadIdx.x);
            int v = k <= nkeys ? first[k] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, v, o);
                if (static_cast<int>(threadIdx.x) >= o) v += up;
            }
            if (k <= nkeys) first[k] = v + carry;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int key = keys[i];
        int before = 0;
        for (int j = 0; j < i; ++j) before += keys[j] == key;
        place[i] = first[key] + before;
    }
    __syncthreads();
}

// One block.  slot[p] = dest * P + (place of pair p among the pairs for rank dest); src[s] = pair in send slot s or -1.
__global__ void __launch_bounds__(kPlanThreads) ep_dispatch_plan_kernel(const int64_t* __restrict__ top_i, int P, int experts, int epr,
                                                                        int world, int32_t* __restrict__ slot, int32_t* __restrict__ src,
                                                                        int* __restrict__ err) {
    extern __shared__ int sh[];
    int* keys = sh;                 // [P]
    int* place = keys + P;          // [P]
    int* first = place + P;         // [experts + 1]
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int64_t e = top_i[p];
        if (e < 0 || e >= experts) {
            if (err) atomicOr(err, LEMOQ_FLAG_BAD_EXPERT);
        }
        keys[p] = static_cast<int>(e < 0 ? 0 : (e >= experts ? experts - 1 : e));
    }
    for (int s = threadIdx.x; s < world * P; s += blockDim.x) src[s] = -1;
    __syncthreads();
    stable_places(keys, P, experts, first, place);
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int dest = keys[p] / epr;
        const int s = dest * P + place[p] - first[dest * epr];
        slot[p] = s;
        src[s] = p;
    }
}

// One block per send slot: the token's row and its expert id, or only the id `experts` for an unused slot.
__global__ void __launch_bounds__(128) ep_dispatch_rows_kernel(const __half* __restrict__ h, const int64_t* __restrict__ top_i,
                                                               const int32_t* __restrict__ src, int K, int H, int experts,
                                                               __half* __restrict__ send) {
    const int s = blockIdx.x, p = src[s];
    __half* row = send + static_cast<int64_t>(s) * (H + kIdCols);
    if (p >= 0) {
        const uint4* from = reinterpret_cast<const uint4*>(h + static_cast<int64_t>(p / K) * H);
        uint4* to = reinterpret_cast<uint4*>(row);
        for (int c = threadIdx.x; c < H / 8; c += blockDim.x) to[c] = from[c];
    }
    if (threadIdx.x == 0) {
        int64_t e = p >= 0 ? top_i[p] : experts;
        if (e < 0 || e > experts) e = experts;
        __half id[kIdCols];
#pragma unroll
        for (int i = 0; i < kIdCols; ++i) id[i] = __float2half_rn(0.f);
        id[0] = __float2half_rn(static_cast<float>(e));  // exact: ids up to 2048
        *reinterpret_cast<uint4*>(row + H) = *reinterpret_cast<const uint4*>(id);
    }
}

// One block.  The R received slots by local expert (padding last): perm[i] = slot of the i-th row, seg[l] = first row
// of local expert l, seg[epr] = number of real rows.
__global__ void __launch_bounds__(kPlanThreads) ep_regroup_plan_kernel(const __half* __restrict__ recv, int R, int H, int experts, int epr,
                                                                       int rank, int32_t* __restrict__ perm, int32_t* __restrict__ seg,
                                                                       int* __restrict__ err) {
    extern __shared__ int sh[];
    int* keys = sh;                 // [R]
    int* place = keys + R;          // [R]
    int* first = place + R;         // [epr + 2]
    for (int s = threadIdx.x; s < R; s += blockDim.x) {
        const int id = static_cast<int>(__half2float(recv[static_cast<int64_t>(s) * (H + kIdCols) + H]));
        int local = id == experts ? epr : id - rank * epr;
        if (local < 0 || local > epr) {  // a row that is not for this rank: treated as padding, and reported
            if (err) atomicOr(err, LEMOQ_FLAG_BAD_EXPERT);
            local = epr;
        }
        keys[s] = local;
    }
    __syncthreads();
    stable_places(keys, R, epr + 1, first, place);
    for (int s = threadIdx.x; s < R; s += blockDim.x) perm[place[s]] = s;
    for (int l = threadIdx.x; l <= epr; l += blockDim.x) seg[l] = first[l];
}

// One block per row of the expert-ordered input: the activations of slot perm[i], zeros behind the real rows.
__global__ void __launch_bounds__(128) ep_regroup_rows_kernel(const __half* __restrict__ recv, const int32_t* __restrict__ perm,
                                                              const int32_t* __restrict__ seg, int epr, int H, __half* __restrict__ x_sorted) {
    const int i = blockIdx.x;
    uint4* to = reinterpret_cast<uint4*>(x_sorted + static_cast<int64_t>(i) * H);
    if (i < seg[epr]) {
        const uint4* from = reinterpret_cast<const uint4*>(recv + static_cast<int64_t>(perm[i]) * (H + kIdCols));
        for (int c = threadIdx.x; c < H / 8; c += blockDim.x) to[c] = from[c];
    } else {
        for (int c = threadIdx.x; c < H / 8; c += blockDim.x) to[c] = make_uint4(0, 0, 0, 0);
    }
}

// One block per row: the result of row i goes back to the slot its input came in.
__global__ void __launch_bounds__(128) ep_return_rows_kernel(const __half* __restrict__ y_sorted, const int32_t* __restrict__ perm,
                                                             const int32_t* __restrict__ seg, int epr, int H, __half* __restrict__ y) {
    const int i = blockIdx.x;
    if (i >= seg[epr]) return;
    const uint4* from = reinterpret_cast<const uint4*>(y_sorted + static_cast<int64_t>(i) * H);
    uint4* to = reinterpret_cast<uint4*>(y + static_cast<int64_t>(perm[i]) * H);
    for (int c = threadIdx.x; c < H / 8; c += blockDim.x) to[c] = from[c];
}

// One block per token: the routing-weighted sum of its K expert outputs in slot order, products and sums in fp32.
__global__ void __launch_bounds__(256) ep_combine_kernel(const __half* __restrict__ back, const int32_t* __restrict__ slot,
                                                         const __half* __restrict__ top_w, int K, int H, __half* __restrict__ out) {
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
        for (int k = 0; k < K; ++k) {
            const float w = __half2float(top_w[t * K + k]);
            const uint4 v = *(reinterpret_cast<const uint4*>(back + static_cast<int64_t>(slot[t * K + k]) * H) + c);
            const __half* vh = reinterpret_cast<const __half*>(&v);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(acc[i], __fmul_rn(__half2float(vh[i]), w));
        }
        __half o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __float2half_rn(acc[i]);
        *(reinterpret_cast<uint4*>(out + static_cast<int64_t>(t) * H) + c) = *reinterpret_cast<const uint4*>(o);
    }
}

}  // namespace
}  // namespace lemoq

using namespace lemoq;

extern "C" int lemoq_ep_dispatch(const void* h, const int64_t* top_i, int T, int K, int H, int experts, int world, void* send,
                                 int32_t* slot, int32_t* src, int* err_flag, void* stream) {
    LEMOQ_REQUIRE(T > 0 && K > 0 && H > 0 && experts > 0 && world > 0, LEMOQ_ERR_INVALID, "ep_dispatch: bad shape");
    LEMOQ_REQUIRE(experts % world == 0, LEMOQ_ERR_INVALID, "ep_dispatch: experts=%d must divide evenly over %d ranks", experts, world);
    LEMOQ_REQUIRE(H % 8 == 0, LEMOQ_ERR_UNSUPPORTED, "ep_dispatch: H=%d must be a multiple of 8", H);
    LEMOQ_REQUIRE(T * K <= kMaxPlanItems && experts <= kMaxPlanKeys, LEMOQ_ERR_UNSUPPORTED, "ep_dispatch: %d pairs / %d experts exceed %d / %d",
                  T * K, experts, kMaxPlanItems, kMaxPlanKeys);
    LEMOQ_REQUIRE(h && top_i && send && slot && src && aligned16(h) && aligned16(send), LEMOQ_ERR_INVALID, "ep_dispatch: null or unaligned pointer");
    const int P = T * K;
    LaunchCfg lc;
    lc.stream = static_cast<cudaStream_t>(stream);
    const size_t smem = (static_cast<size_t>(2) * P + experts + 1) * sizeof(int);
    int rc = launch_kernel(ep_dispatch_plan_kernel, dim3(1), dim3(kPlanThreads), smem, lc, top_i, P, experts, experts / world, world, slot, src, err_flag);
    if (rc != LEMOQ_OK) return rc;
    return launch_kernel(ep_dispatch_rows_kernel, dim3(world * P), dim3(128), 0, lc, reinterpret_cast<const __half*>(h), top_i,
                         static_cast<const int32_t*>(src), K, H, experts, reinterpret_cast<__half*>(send));
}

extern "C" int lemoq_ep_regroup(const void* recv, int R, int H, int experts, int world, int rank, void* x_sorted, int32_t* perm, int32_t* seg,
                                int* err_flag, void* stream) {
    LEMOQ_REQUIRE(R > 0 && H > 0 && experts > 0 && world > 0 && rank >= 0 && rank < world, LEMOQ_ERR_INVALID, "ep_regroup: bad shape");
    LEMOQ_REQUIRE(experts % world == 0 && H % 8 == 0, LEMOQ_ERR_INVALID, "ep_regroup: experts %% world and H %% 8 must be 0");
    LEMOQ_REQUIRE(R <= kMaxPlanItems && experts <= kMaxPlanKeys, LEMOQ_ERR_UNSUPPORTED, "ep_regroup: %d rows exceed %d", R, kMaxPlanItems);
    LEMOQ_REQUIRE(recv && x_sorted && perm && seg && aligned16(recv) && aligned16(x_sorted), LEMOQ_ERR_INVALID, "ep_regroup: null or unaligned pointer");
    const int epr = experts / world;
    LaunchCfg lc;
    lc.stream = static_cast<cudaStream_t>(stream);
    const size_t smem = (static_cast<size_t>(2) * R + epr + 2) * sizeof(int);
    int rc = launch_kernel(ep_regroup_plan_kernel, dim3(1), dim3(kPlanThreads), smem, lc, reinterpret_cast<const __half*>(recv), R, H, experts, epr,
                           rank, perm, seg, err_flag);
    if (rc != LEMOQ_OK) return rc;
    return launch_kernel(ep_regroup_rows_kernel, dim3(R), dim3(128), 0, lc, reinterpret_cast<const __half*>(recv), static_cast<const int32_t*>(perm),
                         static_cast<const int32_t*>(seg), epr, H, reinterpret_cast<__half*>(x_sorted));
}

extern "C" int lemoq_ep_return(const void* y_sorted, const int32_t* perm, const int32_t* seg, int R, int H, int epr, void* y, void* stream) {
    LEMOQ_REQUIRE(R > 0 && H > 0 && H % 8 == 0 && epr > 0, LEMOQ_ERR_INVALID, "ep_return: bad shape");
    LEMOQ_REQUIRE(y_sorted && perm && seg && y && aligned16(y_sorted) && aligned16(y), LEMOQ_ERR_INVALID, "ep_return: null or unaligned pointer");
    LaunchCfg lc;
    lc.stream = static_cast<cudaStream_t>(stream);
    return launch_kernel(ep_return_rows_kernel, dim3(R), dim3(128), 0, lc, reinterpret_cast<const __half*>(y_sorted), perm, seg, epr, H,
                         reinterpret_cast<__half*>(y));
}

extern "C" int lemoq_ep_combine(const void* back, const int32_t* slot, const void* top_w, int T, int K, int H, void* out, void* stream) {
    LEMOQ_REQUIRE(T > 0 && K > 0 && H > 0 && H % 8 == 0, LEMOQ_ERR_INVALID, "ep_combine: bad shape");
    LEMOQ_REQUIRE(back && slot && top_w && out && aligned16(back) && aligned16(out), LEMOQ_ERR_INVALID, "ep_combine: null or unaligned pointer");
    LaunchCfg lc;
    lc.stream = static_cast<cudaStream_t>(stream);
    return launch_kernel(ep_combine_kernel, dim3(T), dim3(256), 0, lc, reinterpret_cast<const __half*>(back), slot, reinterpret_cast<const __half*>(top_w), K,
                         H, reinterpret_cast<__half*>(out));
}
