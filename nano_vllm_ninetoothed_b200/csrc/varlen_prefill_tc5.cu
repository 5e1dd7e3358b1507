// Variable-length causal prefill attention on the Blackwell tensor cores (tcgen05 + TMEM).
//
// One CTA = one 128-row query tile of one sequence for TWO query heads that share a KV head
// (G = hq/hkv must be even), so every K/V tile fetched serves two S tiles and the two tiles
// keep the tensor pipe busy while the other one is in softmax.
//
//   warps 0-3  softmax group 0 (query head 2p)     one thread per query row == TMEM lane
//   warps 4-7  softmax group 1 (query head 2p+1)
//   warp  8    MMA issuer: a single thread issues every tcgen05.mma and tcgen05.commit
//   warp  9    TMA producer: Q tiles once, then 128-key K and V tiles through 2-stage rings
//
//   TMEM (512 columns x 128 lanes, fp32):  S0 [0,128)  S1 [128,256)  O0 [256,384)  O1 [384,512)
//   P (16-bit) overwrites the first 64 columns of its S tile and is read by the PV MMA
//   directly from TMEM as the A operand; V is the MN-major B operand straight from the
//   128-byte-swizzled tile TMA wrote.
//
//   per KV tile j:   S_t = Q_t K_j^T  ->  softmax group t: row max, lazy rescale of O_t,
//                    P_t = exp2(S_t*c - m)  ->  O_t += P_t V_j
//   issue order:     S0(0) S1(0) | PV0(j) S0(j+1) PV1(j) S1(j+1) | ...
//
// Softmax state is per thread (a thread owns a whole row), so there are no shuffles.  The
// running maximum is only raised when it grows by more than 2^8 (O and l stay consistent
// with the stale maximum, P stays below 256), which makes the O rescale rare.
// Every mbarrier wait is bounded; on a timeout the roles fall through to the common exit,
// which frees the tensor memory.
#include <math.h>
#include <stdlib.h>

#include <type_traits>

#include "prefill_internal.h"
#include "tcgen05.cuh"

namespace b200mops {
namespace {

constexpr int kBM = 128;                 // query rows per tile
constexpr int kBN = 128;                 // keys per KV tile
constexpr int kD = 128;                  // head dim
constexpr int kHalf = 128 * 128;         // bytes of one [128 x 64] 16-bit swizzled tile
constexpr int kTileBytes = 2 * kHalf;    // a [128 x 128] operand = two halves
constexpr int kKVStages = 2;
constexpr int kSoftmaxThreads = 256;
constexpr int kMmaWarp = 8, kLoadWarp = 9;
constexpr int kThreads = 320;
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.f;  // log2 units

// shared memory map (offsets from the 1024-aligned base)
constexpr int kOffQ = 0;                                   // 2 tiles
constexpr int kOffK = kOffQ + 2 * kTileBytes;              // kKVStages tiles
constexpr int kOffV = kOffK + kKVStages * kTileBytes;
constexpr int kOffBar = kOffV + kKVStages * kTileBytes;
// barriers: q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2],
//           p_full[2], o_done
constexpr int kNumBars = 1 + 4 * kKVStages + 2 + 2 + 1;
constexpr int kSmemBytes = 1024 + kOffBar + kNumBars * 8 + 16;

#ifdef B200MOPS_TC5_TRACE
// Development aid (not compiled by default): CTA (0,0,0) stamps clock64 at phase boundaries.
__device__ long long g_tc5_trace[3][32][8];
#define TC5_TRACE(role, j, slot)                                                        \
    do {                                                                                \
        if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (j) < 32)          \
            g_tc5_trace[role][j][slot] = clock64();                                     \
    } while (0)
#else
#define TC5_TRACE(role, j, slot) do {} while (0)
#endif

struct Tc5Params {
    void* out; int64_t out_stride_t, out_stride_h;
    const int32_t* cu_q; const int32_t* cu_k;
    int group, causal;
    float scale_log2;
    int32_t* status;
};

template <typename T, int kPolyMask>
__global__ void __launch_bounds__(kThreads, 1)
varlen_prefill_tc5_kernel(const __grid_constant__ CUtensorMap tm_q,
                          const __grid_constant__ CUtensorMap tm_k,
                          const __grid_constant__ CUtensorMap tm_v, const Tc5Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~uintptr_t(1023));
    const uint32_t sbase = smem_u32(smem);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * i; };
    constexpr int Q_FULL = 0, K_FULL = 1, K_EMPTY = K_FULL + kKVStages, V_FULL = K_EMPTY + kKVStages,
                  V_EMPTY = V_FULL + kKVStages, S_FULL = V_EMPTY + kKVStages, P_FULL = S_FULL + 2,
                  O_DONE = P_FULL + 2;

    const int pair = blockIdx.y, b = blockIdx.z;
    const int hq0 = pair * 2;
    const int hk = hq0 / p.group;
    const int q_begin = __ldg(p.cu_q + b), len_q = __ldg(p.cu_q + b + 1) - q_begin;
    const int k_begin = __ldg(p.cu_k + b), len_k = __ldg(p.cu_k + b + 1) - k_begin;
    const int m_tiles = (len_q + kBM - 1) / kBM;
    if ((int)blockIdx.x >= m_tiles) return;
    // Once any CTA of this stream of work has given up on a wait, the rest leave at once
    // instead of each spending its own time limit.
    if (p.status && (*reinterpret_cast<volatile int32_t*>(p.status) & B200MOPS_DEV_WAIT_TIMEOUT)) return;
    const int m0 = (m_tiles - 1 - (int)blockIdx.x) * kBM;     // heavy (late) row tiles first
    const int off = len_k - len_q;
    int n_end = len_k;
    if (p.causal) n_end = min(len_k, m0 + kBM + off);
    const int ntiles = n_end > 0 ? (n_end + kBN - 1) / kBN : 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(bar(Q_FULL), 1);
        for (int s = 0; s < kKVStages; ++s) {
            mbar_init(bar(K_FULL + s), 1);
            mbar_init(bar(K_EMPTY + s), 1);
            mbar_init(bar(V_FULL + s), 1);
            mbar_init(bar(V_EMPTY + s), 1);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(bar(S_FULL + t), 1);
            mbar_init(bar(P_FULL + t), 4);      // one arrival per softmax warp
        }
        mbar_init(bar(O_DONE), 1);
        mbar_fence_init();
    }
    if (warp == kMmaWarp) {
        tc5::tmem_alloc(smem_u32(tmem_slot), kTmemCols);
        tc5::tmem_relinquish();
    }
    tc5::fence_before_sync();
    __syncthreads();
    tc5::fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == kLoadWarp) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0 && ntiles > 0) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_v);
            mbar_arrive_expect_tx(bar(Q_FULL), 2 * kTileBytes);
            for (int t = 0; t < 2; ++t) {
                const uint32_t dst = sbase + kOffQ + t * kTileBytes;
                tma_load_4d(dst, &tm_q, bar(Q_FULL), 0, hq0 + t, q_begin + m0, 0);
                tma_load_4d(dst + kHalf, &tm_q, bar(Q_FULL), 64, hq0 + t, q_begin + m0, 0);
            }
            for (int j = 0; j < ntiles; ++j) {
                const int s = j % kKVStages, round = j / kKVStages;
                const int row = k_begin + j * kBN;
                if (round > 0 && !mbar_wait(bar(K_EMPTY + s), (uint32_t)(round - 1) & 1u, p.status)) break;
                mbar_arrive_expect_tx(bar(K_FULL + s), kTileBytes);
                tma_load_4d(sbase + kOffK + s * kTileBytes, &tm_k, bar(K_FULL + s), 0, hk, row, 0);
                tma_load_4d(sbase + kOffK + s * kTileBytes + kHalf, &tm_k, bar(K_FULL + s), 64, hk, row, 0);
                if (round > 0 && !mbar_wait(bar(V_EMPTY + s), (uint32_t)(round - 1) & 1u, p.status)) break;
                mbar_arrive_expect_tx(bar(V_FULL + s), kTileBytes);
                tma_load_4d(sbase + kOffV + s * kTileBytes, &tm_v, bar(V_FULL + s), 0, hk, row, 0);
                tma_load_4d(sbase + kOffV + s * kTileBytes + kHalf, &tm_v, bar(V_FULL + s), 64, hk, row, 0);
            }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------ MMA issuer
        // The whole warp runs this loop so that descriptor arithmetic stays warp-uniform (it can
        // live in uniform registers); one elected lane executes the tcgen05 instructions.  The
        // issuing thread is the pacemaker of the tensor pipe: every cycle it spends between two
        // tcgen05.mma is a cycle the pipe may idle, so nothing here is recomputed per MMA.
        if (ntiles > 0) {
            constexpr int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
            constexpr uint32_t idesc_s = tc5::instr_desc_f16(fmt, kBM, kBN, 0, 0);
            constexpr uint32_t idesc_o = tc5::instr_desc_f16(fmt, kBM, kD, 0, 1);
            const bool leader = tc5::elect_one();
            const uint32_t tm = __shfl_sync(0xffffffffu, tmem, 0);
            const uint64_t dq = tc5::smem_desc_sw128(sbase + kOffQ, 16, 1024);
            const uint64_t dk = tc5::smem_desc_sw128(sbase + kOffK, 16, 1024);
            const uint64_t dv = tc5::smem_desc_sw128(sbase + kOffV, kHalf, 1024);
            auto wait = [&](int b, uint32_t parity) {
                const bool done = mbar_wait(bar(b), parity, p.status);
                return __all_sync(0xffffffffu, done);
            };
            // S_t = Q_t K_j^T : 8 k-steps of 16 over head_dim, both operands K-major
            auto issue_s = [&](int t, int j) {
                const uint64_t a0 = dq + ((uint32_t)(t * kTileBytes) >> 4);
                const uint64_t b0 = dk + ((uint32_t)((j % kKVStages) * kTileBytes) >> 4);
                if (leader) {
#pragma unroll
                    for (int ks = 0; ks < kD / 16; ++ks) {
                        const uint32_t o = (uint32_t)((ks >> 2) * kHalf + (ks & 3) * 32) >> 4;
                        tc5::mma_ss(tm + t * kBN, a0 + o, b0 + o, idesc_s, ks > 0);
                    }
                    tc5::commit(bar(S_FULL + t));
                }
            };
            // O_t += P_t V_j : 8 k-steps of 16 keys; A = P from TMEM, B = V MN-major
            auto issue_pv = [&](int t, int j) {
                const uint64_t b0 = dv + ((uint32_t)((j % kKVStages) * kTileBytes) >> 4);
                const uint32_t acc0 = j > 0 ? 1u : 0u;
                if (leader) {
#pragma unroll
                    for (int kk = 0; kk < kBN / 16; ++kk)
                        tc5::mma_ts(tm + 256 + t * kD, tm + t * kBN + kk * 8,
                                    b0 + (uint32_t)(kk * 2048 >> 4), idesc_o, kk > 0 ? 1u : acc0);
                }
            };
            bool ok = wait(Q_FULL, 0) && wait(K_FULL + 0, 0);
            if (ok) {
                tc5::fence_after_sync();
                TC5_TRACE(2, 31, 0);
                issue_s(0, 0);
                TC5_TRACE(2, 31, 1);
                issue_s(1, 0);
                TC5_TRACE(2, 31, 2);
                if (leader) tc5::commit(bar(K_EMPTY + 0));
            }
            for (int j = 0; ok && j < ntiles; ++j) {
                const int s = j % kKVStages, sn = (j + 1) % kKVStages;
                const uint32_t ph = (uint32_t)(j / kKVStages) & 1u;
                const uint32_t phn = (uint32_t)((j + 1) / kKVStages) & 1u;
                const bool more = j + 1 < ntiles;
                TC5_TRACE(2, j, 6);
                if (!(ok = wait(V_FULL + s, ph))) break;
                if (!(ok = wait(P_FULL + 0, (uint32_t)j & 1u))) break;
                TC5_TRACE(2, j, 0);
                tc5::fence_after_sync();
                issue_pv(0, j);
                TC5_TRACE(2, j, 1);
                if (more) {
                    if (!(ok = wait(K_FULL + sn, phn))) break;
                    tc5::fence_after_sync();
                    issue_s(0, j + 1);
                }
                TC5_TRACE(2, j, 2);
                if (!(ok = wait(P_FULL + 1, (uint32_t)j & 1u))) break;
                TC5_TRACE(2, j, 3);
                tc5::fence_after_sync();
                issue_pv(1, j);
                if (leader) tc5::commit(bar(V_EMPTY + s));
                TC5_TRACE(2, j, 4);
                if (more) {
                    issue_s(1, j + 1);
                    if (leader) tc5::commit(bar(K_EMPTY + sn));
                }
                TC5_TRACE(2, j, 5);
            }
            if (leader) tc5::commit(bar(O_DONE));
        }
    } else {
        // ------------------------------------------------------------ softmax groups
        const int t = warp >> 2;                        // tile / query head within the pair
        const int row = threadIdx.x & 127;              // query row in the tile == TMEM lane
        const uint32_t lane_base = (uint32_t)(32 * (warp & 3)) << 16;
        const uint32_t tS = tmem + lane_base + t * kBN;
        const uint32_t tO = tmem + lane_base + 256 + t * kD;
        const int qi = m0 + row;                        // sequence-local query index
        const int lim = p.causal ? min(len_k - 1, qi + off) : len_k - 1;   // last visible key
        const float c = p.scale_log2;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        uint32_t sv[kBN / 32][32];
        for (int j = 0; j < ntiles; ++j) {
            ok = mbar_wait(bar(S_FULL + t), (uint32_t)j & 1u, p.status);
            if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
            if (threadIdx.x % 128 == 0) TC5_TRACE(t, j, 0);
            tc5::fence_after_sync();
            const int key0 = j * kBN;
            const bool need_mask = key0 + kBN - 1 > lim;      // this row crosses its limit here
            const bool warp_mask = __any_sync(0xffffffffu, need_mask);
            // The whole S row (128 fp32) is pulled into registers with one wait: TMEM load
            // latency is paid once per tile instead of once per chunk.
#pragma unroll
            for (int cc = 0; cc < kBN / 32; ++cc) tc5::ld32(tS + cc * 32, sv[cc]);
            tc5::wait_ld();
            if (threadIdx.x % 128 == 0) TC5_TRACE(t, j, 1);
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
            if (warp_mask) {
#pragma unroll
                for (int cc = 0; cc < kBN / 32; ++cc)
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (key0 + cc * 32 + i > lim) sv[cc][i] = 0xff800000u;   // -inf
            }
#pragma unroll
            for (int cc = 0; cc < kBN / 32; ++cc)
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    mx0 = tc5::max3(mx0, __uint_as_float(sv[cc][i]), __uint_as_float(sv[cc][i + 1]));
                    mx1 = tc5::max3(mx1, __uint_as_float(sv[cc][i + 2]), __uint_as_float(sv[cc][i + 3]));
                    mx2 = tc5::max3(mx2, __uint_as_float(sv[cc][i + 4]), __uint_as_float(sv[cc][i + 5]));
                    mx3 = tc5::max3(mx3, __uint_as_float(sv[cc][i + 6]), __uint_as_float(sv[cc][i + 7]));
                }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            const float m_new = fmaxf(m_ref, mx * c);
            const bool grow = m_new > m_ref + kRescaleThreshold;   // also true for the first finite max
            if (__any_sync(0xffffffffu, grow)) {
                const float corr = grow ? fast_exp2(m_ref - m_new) : 1.f;   // exp2(-inf) = 0
                if (j > 0) {
                    // S(j) complete implies PV(j-1) complete (one thread issues both, in order),
                    // so O_t is at rest until this group hands P(j) over.
#pragma unroll 1
                    for (int cc = 0; cc < kD / 16; ++cc) {
                        uint32_t ov[16];
                        tc5::ld16(tO + cc * 16, ov);
                        tc5::wait_ld();
#pragma unroll
                        for (int i = 0; i < 16; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
                        tc5::st16(tO + cc * 16, ov);
                    }
                }
                l *= corr;
                if (grow) m_ref = m_new;
            }
            const float sub = m_ref == -INFINITY ? 0.f : m_ref;   // fully masked so far: stay finite
            if (threadIdx.x % 128 == 0) TC5_TRACE(t, j, 2);
            // P = exp2(S*c - m) (masked entries are -inf -> 0), row sum, 16-bit P into the S columns
            // Packed fp32x2 arithmetic for the scale/subtract and the row sum; in tiles that need
            // no mask three pairs in eight take the polynomial exp2 on the FMA pipe, which
            // balances it against the special-function unit (masked entries must come out as
            // exact zeros, which only ex2 gives, so masked tiles use ex2 throughout).
            const tc5::f32x2 c2 = tc5::pack_f32x2(c, c), nsub2 = tc5::pack_f32x2(-sub, -sub);
            tc5::f32x2 lsum = tc5::pack_f32x2(0.f, 0.f);
            auto p_chunk = [&](int cc, auto use_poly) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const tc5::f32x2 x = tc5::fma2(
                        tc5::pack_f32x2(__uint_as_float(sv[cc][i]), __uint_as_float(sv[cc][i + 1])), c2, nsub2);
                    float p0, p1;
                    const int k8 = (i >> 1) & 7;
                    if (decltype(use_poly)::value && ((kPolyMask >> k8) & 1)) {
                        tc5::poly_exp2_x2(x, p0, p1);
                    } else {
                        float x0, x1;
                        tc5::unpack_f32x2(x, x0, x1);
                        p0 = fast_exp2(x0);
                        p1 = fast_exp2(x1);
                    }
                    lsum = tc5::add2(lsum, tc5::pack_f32x2(p0, p1));
                    pk[i >> 1] = pack2<T>(p0, p1);
                }
                tc5::st16(tS + cc * 16, pk);
            };
            if (warp_mask) {
#pragma unroll
                for (int cc = 0; cc < kBN / 32; ++cc) p_chunk(cc, std::false_type{});
            } else {
#pragma unroll
                for (int cc = 0; cc < kBN / 32; ++cc) p_chunk(cc, std::true_type{});
            }
            tc5::wait_st();
            tc5::fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(P_FULL + t));
            if (threadIdx.x % 128 == 0) TC5_TRACE(t, j, 3);
            {
                float l0, l1;
                tc5::unpack_f32x2(lsum, l0, l1);
                l += l0 + l1;
            }
        }
        // ------------------------------------------------------------ epilogue
        if (ok && ntiles > 0) {
            ok = mbar_wait(bar(O_DONE), 0, p.status);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            tc5::fence_after_sync();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            T* orow = reinterpret_cast<T*>(p.out) + (int64_t)(q_begin + qi) * p.out_stride_t +
                      (int64_t)(hq0 + t) * p.out_stride_h;
#pragma unroll
            for (int cc = 0; cc < kD / 32; ++cc) {
                if (ntiles > 0) {
                    tc5::ld32(tO + cc * 32, sv[0]);
                    tc5::wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) sv[0][i] = 0u;
                }
                if (qi < len_q) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 w;
                        w.x = pack2<T>(__uint_as_float(sv[0][i]) * inv, __uint_as_float(sv[0][i + 1]) * inv);
                        w.y = pack2<T>(__uint_as_float(sv[0][i + 2]) * inv, __uint_as_float(sv[0][i + 3]) * inv);
                        w.z = pack2<T>(__uint_as_float(sv[0][i + 4]) * inv, __uint_as_float(sv[0][i + 5]) * inv);
                        w.w = pack2<T>(__uint_as_float(sv[0][i + 6]) * inv, __uint_as_float(sv[0][i + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + cc * 32 + i) = w;
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------- common exit
    __syncwarp();
    tc5::fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc5::fence_after_sync();
        tc5::tmem_dealloc(tmem, kTmemCols);
    }
}

}  // namespace

#ifdef B200MOPS_TC5_TRACE
extern "C" int b200mops_debug_tc5_trace(long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, g_tc5_trace, sizeof(g_tc5_trace)) == cudaSuccess ? 0 : 1;
}
#endif

int launch_varlen_prefill_tc5(const b200mops_varlen_prefill_args* a, const CUtensorMap& tm_q,
                              const CUtensorMap& tm_k, const CUtensorMap& tm_v, cudaStream_t st) {
    Tc5Params p;
    p.out = a->out; p.out_stride_t = a->out_stride_t; p.out_stride_h = a->out_stride_h;
    p.cu_q = a->cu_seqlens_q; p.cu_k = a->cu_seqlens_k;
    p.group = (int)(a->hq / a->hkv);
    p.causal = a->causal ? 1 : 0;
    p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
    p.status = a->status_word;
    const dim3 grid((unsigned)((a->max_seqlen_q + kBM - 1) / kBM), (unsigned)(a->hq / 2),
                    (unsigned)a->batch);
    // Pairs (of every eight) whose exp2 runs as a polynomial on the FMA pipe instead of on the
    // special-function unit.  B200MOPS_TC5_POLY (0..4) overrides the default for measurements.
    static const int poly_pairs = [] {
        const char* e = getenv("B200MOPS_TC5_POLY");
        return e ? atoi(e) : 3;
    }();
    auto launch = [&](auto kernel) -> int {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
            cudaSuccess)
            return B200MOPS_ERR_LAUNCH;
        kernel<<<grid, kThreads, kSmemBytes, st>>>(tm_q, tm_k, tm_v, p);
        return launch_status();
    };
#define B200MOPS_TC5_DISPATCH(TYPE)                                                    \
    switch (poly_pairs) {                                                              \
        case 0: return launch(varlen_prefill_tc5_kernel<TYPE, 0x00>);                  \
        case 1: return launch(varlen_prefill_tc5_kernel<TYPE, 0x10>);                  \
        case 2: return launch(varlen_prefill_tc5_kernel<TYPE, 0x22>);                  \
        case 4: return launch(varlen_prefill_tc5_kernel<TYPE, 0xAA>);                  \
        default: return launch(varlen_prefill_tc5_kernel<TYPE, 0x52>);                 \
    }
    if (a->dtype == B200MOPS_BF16) {
        B200MOPS_TC5_DISPATCH(__nv_bfloat16)
    } else {
        B200MOPS_TC5_DISPATCH(__half)
    }
#undef B200MOPS_TC5_DISPATCH
    return launch_status();
}

}  // namespace b200mops
