// f64 GEMM for Linear forward/backward on sm_100a: TMA-staged shared-memory tiles,
// an mbarrier ring between one producer warp and the consumer warps, DMMA
// (mma.sync m16n8k8 f64) from registers, and the bias / ReLU / 1/n / ReLU-mask
// epilogues applied to the accumulators before the single store of C.
//
//   forward   Y  = X · Wᵀ + b      A = X  [M][K] (K-major)   B = W [N][K] (K-major)
//   backward  dX = dY · W          A = dY [M][K] (K-major)   B = W [K][N] (N-major)
//   backward  dW = dYᵀ · X / n     A = dY [K][M] (M-major)   B = X [K][N] (N-major)
// (src/module/linear.rs:44, :68, :63 of the reference.)
//
// Shared-memory tiles are rows of 16 f64 = 128 bytes written by TMA with the
// 128-byte swizzle (16-byte chunk index XOR row%8), so every fragment is read
// with 16-byte shared loads.  The mma k index and, for M-/N-major operands, the
// m/n index of a fragment element are free to permute as long as A and B agree
// on k and the epilogue knows where each accumulator lives; the mappings below
// pick the permutation that makes one 16-byte load deliver two fragment elements.
#include <cudaTypedefs.h>

#include <algorithm>

#include "common.h"
#include "mma_f64.cuh"

namespace rst {
namespace {

constexpr int kBK = 16;            // k extent of a stage: one 128-byte row of f64
constexpr int kRowBytes = 128;
constexpr int kBoxBytes = 16 * kRowBytes;   // 16x16 box of an M-/N-major operand

struct GemmParams {
    double* C;
    const double* bias;
    const double* mask_src;
    double* splitk_ws;      // [splits][M][N] raw partial sums when splits > 1, then [splits][M] column sums
    double* colsum_out;     // [M]: Σ_k A(m,k) / divisor, fused into the M-major-A kernel (db of Linear::backward)
    double* Ct;             // [N][M]: optional transposed copy of C (splits == 1, M-major A, N-major B)
    int* status;
    double divisor;
    long long wait_limit;   // SM cycles a barrier wait may take before the kernel gives up
    long long M, N, K;
    int tiles_m, tiles_n;
    int k_tiles;            // ceil(K / 16)
    int k_tiles_per_split;
    int splits;
    int epilogue;
    int starve;             // self-test: the producer issues no copy, so every consumer wait runs out
    // Tail of a product whose tile count is not a multiple of the SM count: the main launch
    // computes tiles [0, sk_first_tile), one per CTA; the remaining tiles' k-tiles, laid end to
    // end, are cut into equal runs of sk_units k-tiles for the sk_ctas CTAs of a second launch,
    // which store raw partial tiles that streamk_fixup_kernel adds up in k order.  sk_ctas == 0:
    // the main launch computes every tile (or split of a tile).
    int sk_first_tile, sk_ctas, sk_units, sk_slots;
    double* sk_ws;          // [sk_ctas][sk_slots][BM*BN]
};

// Output tile `tile_index` in launch order -> tile coordinates: groups of 8 tile rows share
// their B tiles in L2.
__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile_index, int& tile_m, int& tile_n) {
    constexpr int kGroup = 8;
    const int tiles_per_group = kGroup * p.tiles_n;
    const int group = tile_index / tiles_per_group;
    const int first_m = group * kGroup;
    const int group_rows = min(p.tiles_m - first_m, kGroup);
    const int in_group = tile_index - group * tiles_per_group;
    tile_m = first_m + in_group % group_rows;
    tile_n = in_group / group_rows;
}

__device__ __forceinline__ double apply_epilogue(const GemmParams& p, double v, long long r, long long c) {
    switch (p.epilogue) {
        case kEpiBias: return v + p.bias[c];
        case kEpiBiasRelu: return fmax(v + p.bias[c], 0.0);
        case kEpiDivN: return v / p.divisor;
        case kEpiMask: return v * (p.mask_src[r * p.N + c] > 0.0 ? 1.0 : 0.0);
        default: return v;
    }
}

template <int W> __device__ __forceinline__ void load_run(double (&v)[W], const double* src);
template <> __device__ __forceinline__ void load_run<2>(double (&v)[2], const double* src) {
    const double2 x = *reinterpret_cast<const double2*>(src);
    v[0] = x.x; v[1] = x.y;
}
template <> __device__ __forceinline__ void load_run<4>(double (&v)[4], const double* src) {
    asm volatile("ld.global.v4.f64 {%0,%1,%2,%3}, [%4];" : "=d"(v[0]), "=d"(v[1]), "=d"(v[2]), "=d"(v[3]) : "l"(src));
}
template <int W> __device__ __forceinline__ void store_run(double* dst, const double (&v)[W]);
template <> __device__ __forceinline__ void store_run<2>(double* dst, const double (&v)[2]) {
    *reinterpret_cast<double2*>(dst) = make_double2(v[0], v[1]);
}
template <> __device__ __forceinline__ void store_run<4>(double* dst, const double (&v)[4]) {
    asm volatile("st.global.v4.f64 [%0], {%1,%2,%3,%4};" ::"l"(dst), "d"(v[0]), "d"(v[1]), "d"(v[2]), "d"(v[3]) : "memory");
}

// Finishes W consecutive elements of row r starting at column c0: epilogue, then store.
// With vec_ok (row pitch and bases aligned to the run) whole runs use one 16- or 32-byte
// access per array; ragged edges and unaligned tensors take the element-wise path.
template <int W>
__device__ __forceinline__ void emit_run(const GemmParams& p, long long r, long long c0, double (&v)[W], bool vec_ok) {
    double* dst = p.C + r * p.N + c0;
    if (vec_ok && c0 + W <= p.N) {
        if (p.epilogue == kEpiMask) {
            double m[W];
            load_run<W>(m, p.mask_src + r * p.N + c0);
#pragma unroll
            for (int i = 0; i < W; ++i) v[i] = v[i] * (m[i] > 0.0 ? 1.0 : 0.0);
        } else if (p.epilogue == kEpiBias || p.epilogue == kEpiBiasRelu) {
            double b[W];
            load_run<W>(b, p.bias + c0);
#pragma unroll
            for (int i = 0; i < W; ++i) {
                v[i] = v[i] + b[i];
                if (p.epilogue == kEpiBiasRelu) v[i] = fmax(v[i], 0.0);
            }
        } else if (p.epilogue == kEpiDivN) {
#pragma unroll
            for (int i = 0; i < W; ++i) v[i] = v[i] / p.divisor;
        }
        store_run<W>(dst, v);
    } else {
#pragma unroll
        for (int i = 0; i < W; ++i)
            if (c0 + i < p.N) dst[i] = apply_epilogue(p, v[i], r, c0 + i);
    }
}

template <int BM, int BN, int WARPS_M, int WARPS_N, int STAGES, bool A_K, bool B_K>
struct Cfg {
    static_assert(A_K || !B_K, "M-major A with K-major B is not used by Linear");
    static constexpr int kConsumerWarps = WARPS_M * WARPS_N;
    // With two warpgroups of consumers the producer gets a warpgroup of its own (one working
    // warp, three that leave at once), so that the CTA can move registers from the producer's
    // warpgroup to the consumers' (setmaxnreg works on whole warpgroups).  A CTA of 9 warps is
    // allocated registers as if it had 12 anyway: 168 per thread.  After the move the
    // consumers own 232 each and the producer's warpgroup 40: 256*232 + 128*40 = 64512.
    static constexpr bool kRegSplit = (kConsumerWarps == 8) && (BM == 128);
    static constexpr int kThreads = kRegSplit ? 384 : (kConsumerWarps + 1) * 32;
    static constexpr int kConsumerRegs = 232, kProducerRegs = 40;
    static constexpr int WTM = BM / WARPS_M, WTN = BN / WARPS_N;
    static constexpr int MT = WTM / 16, NT = WTN / 8;
    static_assert(WTM % 16 == 0 && WTN % 16 == 0, "warp tile must be a multiple of 16x16");
    static constexpr int kABytes = BM * kRowBytes;
    static constexpr int kBBytes = BN * kRowBytes;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kSmemBytes = STAGES * kStageBytes + 1024 /*alignment slack*/ + 2 * STAGES * 8;
    // k permutation: both operands M-/N-major -> pairs (2t, 2t+1); otherwise the
    // K-major operand dictates pairs (4t+2i, 4t+2i+1).
    static constexpr bool kMnNatural = !A_K && !B_K;
};

// One CTA's share of one product: output tile `tile_index` (in the grouped order below),
// k range of split `split`.  tmA and tmB must refer to kernel parameters declared
// __grid_constant__ (the TMA unit reads the descriptors through their address).
template <int BM, int BN, int WARPS_M, int WARPS_N, int STAGES, bool A_K, bool B_K, bool FUSE_COLSUM,
          bool WRITE_T = false, bool STREAMED = false>
__device__ __forceinline__ void gemm_tile(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p,
                                          const int tile_index, const int split) {
    using C_ = Cfg<BM, BN, WARPS_M, WARPS_N, STAGES, A_K, B_K>;
    constexpr int MT = C_::MT, NT = C_::NT;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = smem_base + STAGES * C_::kStageBytes;   // full[STAGES], empty[STAGES]
    auto full_bar = [&](int s) { return bars + (uint32_t)s * 8u; };
    auto empty_bar = [&](int s) { return bars + (uint32_t)(STAGES + s) * 8u; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // The work of this CTA is a short list of segments (tile, k range): one for a CTA that owns
    // a tile (or a split of it), up to sk_slots for a CTA of the streamed tail.  The producer
    // and the consumers walk the same list; the stage ring runs on across segments.
    // STREAMED is a kernel of its own (the tail launch): in the ordinary kernel the segment list
    // has one entry and all of this folds away.
    constexpr bool streamed = STREAMED;
    // Segment number `seg` of this CTA, derived from scratch each time so that nothing but
    // `seg` stays live across the main loop.  CTA x of the tail launch owns the run that starts
    // at k-tile x * sk_units of the tail laid end to end (31 bits suffice, the host checks).
    int seg = 0, seg_tile = 0, kt_begin = 0, kt_end = 0;
    auto next_segment = [&]() -> bool {
        if (!streamed) {
            if (seg > 0) return false;
            seg_tile = tile_index;
            kt_begin = split * p.k_tiles_per_split;
            kt_end = min(kt_begin + p.k_tiles_per_split, p.k_tiles);
        } else {
            const int tail_units = (p.tiles_m * p.tiles_n - p.sk_first_tile) * p.k_tiles;
            const int u0 = tile_index * p.sk_units;
            const int u1 = min(u0 + p.sk_units, tail_units);
            const int t = u0 / p.k_tiles + seg;              // tile of the tail this segment lies in
            const int lo = max(u0, t * p.k_tiles), hi = min(u1, (t + 1) * p.k_tiles);
            if (lo >= hi) return false;
            seg_tile = p.sk_first_tile + t;
            kt_begin = lo - t * p.k_tiles;
            kt_end = hi - t * p.k_tiles;
        }
        ++seg;
        return true;
    };
    int tile_m = 0, tile_n = 0, m0 = 0, n0 = 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), C_::kConsumerWarps);
        }
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncthreads();
    // Everything above touched shared memory and parameters only; from here on the kernel
    // reads operands and writes results that the grid launched before it may still be
    // using.
    grid_dependency_release();
    grid_dependency_wait();

    if (warp >= C_::kConsumerWarps) {
        // ---------------- producer warp: one lane drives TMA ----------------
        if (C_::kRegSplit) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C_::kProducerRegs));
        if (warp == C_::kConsumerWarps && lane == 0 && !p.starve) {
            tma_prefetch_desc(&tmA);
            tma_prefetch_desc(&tmB);
            int it = 0;
            bool alive = true;
            while (alive && next_segment()) {
              tile_coords(p, seg_tile, tile_m, tile_n);
              m0 = tile_m * BM; n0 = tile_n * BN;
              for (int kt = kt_begin; kt < kt_end; ++kt, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                if (!mbar_wait_bounded(empty_bar(s), ph ^ 1u, p.wait_limit)) {
                    atomicExch(p.status, kDevBarrierTimeout);
                    atomicExch(p.status + 1, 1);
                    alive = false;
                    break;
                }
                mbar_expect_tx(full_bar(s), C_::kStageBytes);
                const uint32_t As = smem_base + (uint32_t)s * C_::kStageBytes;
                const uint32_t Bs = As + C_::kABytes;
                const int k0 = kt * kBK;
                if (A_K) {
                    tma_load_2d(As, &tmA, k0, m0, full_bar(s));
                } else {
#pragma unroll
                    for (int j = 0; j < BM / 16; ++j)
                        tma_load_2d(As + j * kBoxBytes, &tmA, m0 + j * 16, k0, full_bar(s));
                }
                if (B_K) {
                    tma_load_2d(Bs, &tmB, k0, n0, full_bar(s));
                } else {
#pragma unroll
                    for (int j = 0; j < BN / 16; ++j)
                        tma_load_2d(Bs + j * kBoxBytes, &tmB, n0 + j * 16, k0, full_bar(s));
                }
              }
            }
        }
        return;
    }

    // ---------------- consumer warps ----------------
    if (C_::kRegSplit) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C_::kConsumerRegs));
    const int wm = warp / WARPS_N, wn = warp % WARPS_N;
    const int g = lane >> 2, t = lane & 3;

    double acc[MT][NT][4];

    // Column sums of the M-major A operand (db = Σ_rows dY / n, linear.rs:65-67): the
    // warps of the first tile column that hold the A fragments anyway add them up.
    static_assert(!FUSE_COLSUM || !A_K, "column sums are taken from an M-major A operand");
    bool do_colsum = false;
    double asum[FUSE_COLSUM ? MT : 1][2];

    // Per-thread byte offsets inside a stage that do not depend on the k sub-step.
    // K-major operand: row*128, chunk (2t+i) ^ (row%8) with row%8 == g.
    const uint32_t a_row_off = (uint32_t)(wm * C_::WTM + g) * kRowBytes;          // + mt*16*128 (+8 rows: +1024)
    const uint32_t b_row_off = (uint32_t)(wn * C_::WTN + g) * kRowBytes;          // + nt*8*128
    const uint32_t kchunk0 = (uint32_t)((2 * t) ^ g) << 4;                        // i = 0; i = 1 flips bit 4
    // M-/N-major operand: box base + k*128 + ((g ^ k%8) << 4)
    const uint32_t a_box_off = (uint32_t)(wm * C_::WTM / 16) * kBoxBytes;         // + mt*2048
    const uint32_t b_box_off = (uint32_t)(wn * C_::WTN / 16) * kBoxBytes;         // + (nt/2)*2048

    // Rows of an M-/N-major tile that feed logical k = t and k = t+4 of sub-step i, as
    // byte offsets inside a box; computed once, outside the k loop.
    uint32_t mn_off[2][2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int kr0 = C_::kMnNatural ? (8 * i + 2 * t) : (4 * t + 2 * i);
        const int kr1 = kr0 + 1;
        mn_off[i][0] = (uint32_t)kr0 * kRowBytes + ((uint32_t)(g ^ (kr0 & 7)) << 4);
        mn_off[i][1] = (uint32_t)kr1 * kRowBytes + ((uint32_t)(g ^ (kr1 & 7)) << 4);
    }

    // Fragments of k sub-step i (0 or 1) of the stage at (As, Bs).
    auto load_frags = [&](uint32_t As, uint32_t Bs, int i, double (&a)[MT][4], double (&b)[NT][2]) {
        const uint32_t mn_off0 = mn_off[i][0], mn_off1 = mn_off[i][1];
        const uint32_t kchunk = kchunk0 ^ ((uint32_t)i << 4);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            if (A_K) {
                const uint32_t addr = As + a_row_off + (uint32_t)mt * 16 * kRowBytes + kchunk;
                lds128(a[mt][0], a[mt][2], addr);                 // row g   : k = t, t+4
                lds128(a[mt][1], a[mt][3], addr + 8 * kRowBytes); // row g+8
            } else {
                const uint32_t box = As + a_box_off + (uint32_t)mt * kBoxBytes;
                lds128(a[mt][0], a[mt][1], box + mn_off0);        // k = t   : m = 2g, 2g+1
                lds128(a[mt][2], a[mt][3], box + mn_off1);        // k = t+4
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            if (B_K) {
                const uint32_t addr = Bs + b_row_off + (uint32_t)nt * 8 * kRowBytes + kchunk;
                lds128(b[nt][0], b[nt][1], addr);                 // n = g : k = t, t+4
            } else if ((nt & 1) == 0) {
                const uint32_t box = Bs + b_box_off + (uint32_t)(nt / 2) * kBoxBytes;
                lds128(b[nt][0], b[nt + 1][0], box + mn_off0);    // k = t   : n = 2g (even tile), 2g+1 (odd tile)
                lds128(b[nt][1], b[nt + 1][1], box + mn_off1);    // k = t+4
            }
        }
    };
    auto multiply = [&](const double (&a)[MT][4], const double (&b)[NT][2]) {
        if (FUSE_COLSUM) {
            if (do_colsum) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    asum[mt][0] += a[mt][0] + a[mt][2];           // m = 2g
                    asum[mt][1] += a[mt][1] + a[mt][3];           // m = 2g+1
                }
            }
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) dmma_m16n8k8(acc[mt][nt], a[mt], b[nt]);
    };
    auto wait_full = [&](int it) -> bool {
        if (mbar_wait_bounded(full_bar(it % STAGES), (uint32_t)(it / STAGES) & 1u, p.wait_limit)) return true;
        atomicExch(p.status, kDevBarrierTimeout);
        atomicExch(p.status + 1, 2);
        return false;       // results are invalid from here on
    };
    // The stage is about to be rewritten by TMA (async proxy) after having been read
    // with ordinary shared loads (generic proxy): every reader orders its reads against
    // the async proxy before the warp releases the stage.  Without this fence, refilled
    // stages were observed half-written on B200.
    auto release = [&](int it) {
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(it % STAGES));
    };
    auto stage_a = [&](int it) { return smem_base + (uint32_t)(it % STAGES) * C_::kStageBytes; };

    bool ok = true;
    int it = 0;                           // stages consumed so far, over all segments
  while (ok && next_segment()) {
    tile_coords(p, seg_tile, tile_m, tile_n);
    m0 = tile_m * BM; n0 = tile_n * BN;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[mt][nt][e] = 0.0;
    do_colsum = FUSE_COLSUM && p.colsum_out != nullptr && tile_n == 0 && wn == 0;
#pragma unroll
    for (int mt = 0; mt < (FUSE_COLSUM ? MT : 1); ++mt) asum[mt][0] = asum[mt][1] = 0.0;

    for (const int it_end = it + (kt_end - kt_begin); it < it_end; ++it) {
        if (!wait_full(it)) { ok = false; break; }
        const uint32_t As = stage_a(it);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            double a[MT][4], b[NT][2];
            load_frags(As, As + C_::kABytes, i, a, b);
            multiply(a, b);
        }
        release(it);
    }

    // ---------------- epilogue: registers -> global ----------------
    // Coordinates of accumulator element (mt, h, nt, e): h selects logical row g or g+8.
    auto row_of = [&](int mt, int h) -> long long {
        return m0 + wm * C_::WTM + mt * 16 + (A_K ? (g + 8 * h) : (2 * g + h));
    };
    auto col_of = [&](int nt, int e) -> long long {
        if (B_K) return n0 + wn * C_::WTN + nt * 8 + 2 * t + e;
        return n0 + wn * C_::WTN + (nt & ~1) * 8 + 4 * t + 2 * e + (nt & 1);
    };
    if (FUSE_COLSUM) {
        if (do_colsum) {      // warp-uniform: add the four lanes that share g
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    double v = asum[mt][h];
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    asum[mt][h] = v;
                }
        }
    }

    const long long MN = p.M * p.N;
    if (streamed) {
        // raw partial tile, addressed inside the tile; the fix-up kernel adds the runs of a
        // tile in k order and applies the epilogue
        double* part = p.sk_ws + ((long long)tile_index * p.sk_slots + (seg - 1)) * (BM * BN);
        if (ok) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    double* prow = part + (int)(row_of(mt, h) - m0) * BN;
                    // the same runs of consecutive columns as in the final store: 16- and 32-byte stores
                    if (B_K) {
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            double v[2] = {acc[mt][nt][2 * h], acc[mt][nt][2 * h + 1]};
                            store_run<2>(prow + (int)(col_of(nt, 0) - n0), v);
                        }
                    } else {
#pragma unroll
                        for (int nt = 0; nt < NT; nt += 2) {
                            double v[4] = {acc[mt][nt][2 * h], acc[mt][nt + 1][2 * h], acc[mt][nt][2 * h + 1],
                                           acc[mt][nt + 1][2 * h + 1]};
                            store_run<4>(prow + (int)(col_of(nt, 0) - n0), v);
                        }
                    }
                }
        }
        continue;
    }
    if (p.splits == 1) {
        constexpr int kRun = B_K ? 2 : 4;
        const bool vec_ok = (p.N % kRun == 0) &&
                            ((((uintptr_t)p.C | (uintptr_t)p.mask_src | (uintptr_t)p.bias) & (8 * kRun - 1)) == 0);
        if (ok) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const long long r = row_of(mt, h);
                    if (r >= p.M) continue;
                    // A thread owns runs of consecutive columns in a row: two per n-tile with
                    // a K-major B, four per pair of n-tiles with an N-major B.  Each run is
                    // finished (bias or mask loaded first, then one vector store) on its own,
                    // so the epilogue's loads do not queue behind its stores.
                    if (B_K) {
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            double v[2] = {acc[mt][nt][2 * h], acc[mt][nt][2 * h + 1]};
                            emit_run<2>(p, r, col_of(nt, 0), v, vec_ok);
                        }
                    } else {
#pragma unroll
                        for (int nt = 0; nt < NT; nt += 2) {
                            double v[4] = {acc[mt][nt][2 * h], acc[mt][nt + 1][2 * h], acc[mt][nt][2 * h + 1],
                                           acc[mt][nt + 1][2 * h + 1]};
                            emit_run<4>(p, r, col_of(nt, 0), v, vec_ok);
                            if (WRITE_T) {    // keep the finished values for the transposed copy below
                                acc[mt][nt][2 * h] = v[0]; acc[mt][nt + 1][2 * h] = v[1];
                                acc[mt][nt][2 * h + 1] = v[2]; acc[mt][nt + 1][2 * h + 1] = v[3];
                            }
                        }
                    }
                    if (FUSE_COLSUM) {
                        if (do_colsum && t == 0) p.colsum_out[r] = asum[mt][h] / p.divisor;
                    }
                }
            // Second, transposed copy of the finished tile ([N][M] in memory), for a consumer
            // that wants this matrix as an M-major operand (the dX product of the next layer
            // down reads the gradient that way).  A thread holds rows 2g and 2g+1 of a column:
            // one 16-byte store each.  The host asks for it only when the runs above took the
            // vector path (N a multiple of 4, M even, aligned bases), so `acc` holds final values.
            if (WRITE_T) {
                static_assert(!WRITE_T || (!A_K && !B_K), "the transposed copy is written from the M-/N-major layout");
                if (p.Ct != nullptr && vec_ok) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const long long r0 = row_of(mt, 0);
                        if (r0 >= p.M) continue;
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const long long c = col_of(nt, e);
                                if (c < p.N)
                                    *reinterpret_cast<double2*>(p.Ct + c * p.M + r0) =
                                        make_double2(acc[mt][nt][e], acc[mt][nt][2 + e]);
                            }
                    }
                }
            }
        }
        continue;
    }

    // Split-K: every split stores its raw partial tile (and partial column sums);
    // splitk_reduce_kernel adds them in split order and applies the epilogue.
    double* part = p.splitk_ws + (long long)split * MN;
    double* colpart = p.splitk_ws + (long long)p.splits * MN;            // [splits][M]
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const long long r = row_of(mt, h);
            if (r >= p.M) continue;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const long long c = col_of(nt, e);
                    if (c < p.N) part[r * p.N + c] = acc[mt][nt][2 * h + e];
                }
            if (FUSE_COLSUM) {
                if (do_colsum && t == 0) colpart[(long long)split * p.M + r] = asum[mt][h];
            }
        }
  }   // segments
}

template <int BM, int BN, int WARPS_M, int WARPS_N, int STAGES, bool A_K, bool B_K, bool FUSE_COLSUM,
          bool WRITE_T = false>
__global__ void __launch_bounds__((Cfg<BM, BN, WARPS_M, WARPS_N, STAGES, A_K, B_K>::kThreads), 1)
gemm_f64_tma_dmma(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const GemmParams p) {
    gemm_tile<BM, BN, WARPS_M, WARPS_N, STAGES, A_K, B_K, FUSE_COLSUM, WRITE_T>(tmA, tmB, p, (int)blockIdx.x,
                                                                               (int)blockIdx.y);
}

// The tail of a large product (see GemmParams::sk_*): CTA x computes the run of k-tiles
// [x * sk_units, (x+1) * sk_units) of the tail's tiles laid end to end and stores one raw
// partial tile per tile it touches.
template <int BM, int BN, int WARPS_M, int WARPS_N, int STAGES, bool A_K, bool B_K>
__global__ void __launch_bounds__((Cfg<BM, BN, WARPS_M, WARPS_N, STAGES, A_K, B_K>::kThreads), 1)
gemm_f64_tma_dmma_tail(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const GemmParams p) {
    gemm_tile<BM, BN, WARPS_M, WARPS_N, STAGES, A_K, B_K, false, false, true>(tmA, tmB, p, (int)blockIdx.x, 0);
}

// Several independent products of one layout in one launch: the dW (and db) products of
// a chain of small layers, none of which fills the GPU by itself.  CTA x belongs to the
// product i with first_cta[i] <= x < first_cta[i+1]; within a product the CTAs are
// ordered split-major.
constexpr int kMaxGroup = 4;
struct GroupMaps { CUtensorMap a[kMaxGroup], b[kMaxGroup]; };
struct GroupParams {
    int count;
    int first_cta[kMaxGroup + 1];
    GemmParams p[kMaxGroup];
};

template <int BM, int BN, int WARPS_M, int WARPS_N, int STAGES, bool A_K, bool B_K, bool FUSE_COLSUM>
__global__ void __launch_bounds__((Cfg<BM, BN, WARPS_M, WARPS_N, STAGES, A_K, B_K>::kThreads), 1)
gemm_f64_tma_dmma_grouped(const __grid_constant__ GroupMaps maps, const __grid_constant__ GroupParams gp) {
    int i = 0;
    while (i + 1 < gp.count && (int)blockIdx.x >= gp.first_cta[i + 1]) ++i;
    const int local = (int)blockIdx.x - gp.first_cta[i];
    const int tiles = gp.p[i].tiles_m * gp.p[i].tiles_n;
    gemm_tile<BM, BN, WARPS_M, WARPS_N, STAGES, A_K, B_K, FUSE_COLSUM>(maps.a[i], maps.b[i], gp.p[i],
                                                                      local % tiles, local / tiles);
}

// Sums the split-K partials in split order and applies the epilogue; elements past
// M*N are the fused column sums (db).
__device__ __forceinline__ void reduce_splits(const GemmParams& p) {
    const long long MN = p.M * p.N;
    const long long total = MN + (p.colsum_out ? p.M : 0);
    const long long stride = (long long)gridDim.x * blockDim.x;
    const double* colpart = p.splitk_ws + (long long)p.splits * MN;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        double v = 0.0;
        if (i < MN) {
#pragma unroll 4
            for (int z = 0; z < p.splits; ++z) v += p.splitk_ws[(long long)z * MN + i];
            p.C[i] = apply_epilogue(p, v, i / p.N, i % p.N);
        } else {
            const long long m = i - MN;
#pragma unroll 4
            for (int z = 0; z < p.splits; ++z) v += colpart[(long long)z * p.M + m];
            p.colsum_out[m] = v / p.divisor;
        }
    }
}

__global__ void __launch_bounds__(256) splitk_reduce_kernel(const GemmParams p) {
    grid_dependency_release();
    grid_dependency_wait();
    reduce_splits(p);
}

__global__ void __launch_bounds__(256) splitk_reduce_grouped_kernel(const __grid_constant__ GroupParams gp) {
    grid_dependency_release();
    grid_dependency_wait();
    for (int i = 0; i < gp.count; ++i)
        if (gp.p[i].splits > 1) reduce_splits(gp.p[i]);
}

// Adds up the partial tiles of the streamed tail.  Tile `tr` of the tail owns k-tiles
// [tr*k_tiles, (tr+1)*k_tiles) of the tail's run; the CTAs whose runs of sk_units k-tiles
// overlap it each left one partial tile, which are added in k order before the epilogue.
// One block finishes 16 rows of a tile.
template <int BM, int BN>
__global__ void __launch_bounds__(256) streamk_fixup_kernel(const GemmParams p) {
    grid_dependency_release();
    grid_dependency_wait();
    constexpr int kRowBlocks = BM / 16;
    const int tr = (int)blockIdx.x / kRowBlocks, rb = (int)blockIdx.x % kRowBlocks;
    int tile_m, tile_n;
    tile_coords(p, p.sk_first_tile + tr, tile_m, tile_n);
    const long long u_lo = (long long)tr * p.k_tiles, u_hi = u_lo + p.k_tiles - 1;
    const int j_lo = (int)(u_lo / p.sk_units), j_hi = (int)(u_hi / p.sk_units);
    for (int e = threadIdx.x; e < 16 * BN; e += 256) {
        const int lr = rb * 16 + e / BN, lc = e % BN;
        const long long r = (long long)tile_m * BM + lr, c = (long long)tile_n * BN + lc;
        if (r >= p.M || c >= p.N) continue;
        double v = 0.0;
        for (int j = j_lo; j <= j_hi; ++j) {
            const int slot = tr - (int)(((long long)j * p.sk_units) / p.k_tiles);   // the run's first tile is its slot 0
            v += p.sk_ws[((long long)j * p.sk_slots + slot) * (BM * BN) + lr * BN + lc];
        }
        v = apply_epilogue(p, v, r, c);
        p.C[r * p.N + c] = v;
        if (p.Ct != nullptr) p.Ct[c * p.M + r] = v;
    }
}

// Plain-load kernel for operands TMA cannot address (odd row pitch or a base
// that is not 16-byte aligned); shapes like the reference's own 3x2 unit tests.
__global__ void __launch_bounds__(256)
gemm_f64_plain(const double* __restrict__ A, const double* __restrict__ B, long long sam, long long sak,
               long long sbk, long long sbn, const GemmParams p) {
    const long long total = p.M * p.N;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long r = i / p.N, c = i % p.N;
        double v = 0.0;
        for (long long k = 0; k < p.K; ++k) v = fma(A[r * sam + k * sak], B[k * sbk + c * sbn], v);
        p.C[i] = apply_epilogue(p, v, r, c);
    }
}

// Raises a kernel's dynamic shared-memory limit once per context (the attribute belongs to
// the device the context is bound to).
int allow_dynamic_smem(rst_ctx* ctx, const void* kernel, int bytes) {
    if (ctx->smem_attr_done.count(kernel)) return RST_OK;
    RST_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    ctx->smem_attr_done.insert(kernel);
    return RST_OK;
}

int encode_map(rst_ctx* ctx, CUtensorMap* map, const double* base, long long inner, long long outer,
               int box_inner, int box_outer) {
    auto fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ctx->encode_tiled);
    cuuint64_t gdim[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t gstride[1] = {(cuuint64_t)inner * sizeof(double)};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 2, const_cast<double*>(base), gdim, gstride, box,
                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(ctx, RST_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d (inner %lld, outer %lld)",
                    (int)r, inner, outer);
    return RST_OK;
}

template <int BM, int BN, int WARPS_M, int WARPS_N, int STAGES, bool A_K, bool B_K, bool FUSE_COLSUM,
          bool WRITE_T = false>
int launch_cfg(rst_ctx* ctx, const GemmArgs& a, GemmParams& p, int splits) {
    using C_ = Cfg<BM, BN, WARPS_M, WARPS_N, STAGES, A_K, B_K>;
    auto kernel = gemm_f64_tma_dmma<BM, BN, WARPS_M, WARPS_N, STAGES, A_K, B_K, FUSE_COLSUM, WRITE_T>;
    RST_TRY(allow_dynamic_smem(ctx, reinterpret_cast<const void*>(kernel), C_::kSmemBytes));
    CUtensorMap tmA, tmB;
    if (A_K) RST_TRY(encode_map(ctx, &tmA, a.A, a.K, a.M, kBK, BM));
    else     RST_TRY(encode_map(ctx, &tmA, a.A, a.M, a.K, 16, kBK));
    if (B_K) RST_TRY(encode_map(ctx, &tmB, a.B, a.K, a.N, kBK, BN));
    else     RST_TRY(encode_map(ctx, &tmB, a.B, a.N, a.K, 16, kBK));

    p.tiles_m = (int)((a.M + BM - 1) / BM);
    p.tiles_n = (int)((a.N + BN - 1) / BN);
    p.k_tiles = (int)((a.K + kBK - 1) / kBK);
    p.splits = splits;
    p.k_tiles_per_split = (p.k_tiles + splits - 1) / splits;
    if (p.k_tiles_per_split < 1) p.k_tiles_per_split = 1;
    p.splits = std::max(1, (p.k_tiles + p.k_tiles_per_split - 1) / p.k_tiles_per_split);
    if (p.splits > 1) {
        size_t need = (size_t)p.splits * ((size_t)a.M * (size_t)a.N + (size_t)a.M) * sizeof(double);
        RST_TRY(ensure_scratch(ctx, (void**)&ctx->splitk_ws, &ctx->splitk_ws_bytes, need, "split-K"));
        p.splitk_ws = ctx->splitk_ws;
    }
    p.colsum_out = FUSE_COLSUM ? a.colsum_out : nullptr;
    // A large product whose tiles do not fill the last wave (4096 tiles on 148 SMs: 27.7 waves,
    // the last one two thirds full) hands the k-tiles of that wave's tiles out in equal runs,
    // one per SM, so that all SMs finish together; a fix-up kernel adds the runs of a tile.
    long long ctas_x = (long long)p.tiles_m * p.tiles_n;
    p.sk_ctas = 0;
    if (BM == 128 && !FUSE_COLSUM && p.splits == 1 && ctx->stream_tail && !a.starve_producer) {
        const long long tiles = ctas_x, rest = tiles % ctx->num_sms;
        const long long units = (rest * p.k_tiles + ctx->num_sms - 1) / ctx->num_sms;
        // what the tail launch saves, in k-tile times per SM: the idle share of the last wave; what
        // it costs: a second prologue, two partial-tile stores per CTA and the fix-up, about 100 of
        // them (measured: 8192x4096x4096 with 41 to save broke even, 8192^3 with 166 gained 0.6 %)
        const long long saved = (ctx->num_sms - rest) * p.k_tiles / ctx->num_sms;
        if (tiles >= 2LL * ctx->num_sms && rest > 0 && saved >= 100 && units >= 16 &&
            (rest + 1) * p.k_tiles < 0x7fffffffLL) {
            p.sk_first_tile = (int)(tiles - rest);
            p.sk_ctas = ctx->num_sms;
            p.sk_units = (int)units;
            p.sk_slots = (int)((units + p.k_tiles - 1) / p.k_tiles) + 1;
            size_t need = (size_t)p.sk_ctas * (size_t)p.sk_slots * (size_t)(BM * BN) * sizeof(double);
            RST_TRY(ensure_scratch(ctx, (void**)&ctx->splitk_ws, &ctx->splitk_ws_bytes, need, "tail-run"));
            p.sk_ws = ctx->splitk_ws;
            ctas_x = p.sk_first_tile;
        }
    }
    dim3 grid((unsigned)ctas_x, (unsigned)p.splits);
    launch_step_kernel(ctx, ctx->compute, kernel, grid, dim3(C_::kThreads), (size_t)C_::kSmemBytes, tmA, tmB, p);
    RST_TRY(after_launch(ctx, "gemm_f64_tma_dmma"));
    if (p.sk_ctas > 0) {
        auto tail = gemm_f64_tma_dmma_tail<BM, BN, WARPS_M, WARPS_N, STAGES, A_K, B_K>;
        RST_TRY(allow_dynamic_smem(ctx, reinterpret_cast<const void*>(tail), C_::kSmemBytes));
        launch_step_kernel(ctx, ctx->compute, tail, dim3((unsigned)p.sk_ctas), dim3(C_::kThreads),
                           (size_t)C_::kSmemBytes, tmA, tmB, p);
        RST_TRY(after_launch(ctx, "gemm_f64_tma_dmma_tail"));
        const unsigned blocks = (unsigned)((p.tiles_m * p.tiles_n - p.sk_first_tile) * (BM / 16));
        launch_step_kernel(ctx, ctx->compute, streamk_fixup_kernel<BM, BN>, dim3(blocks), dim3(256), 0, p);
        RST_TRY(after_launch(ctx, "streamk_fixup_kernel"));
    }
    if (p.splits > 1) {
        const long long total = a.M * a.N + (p.colsum_out ? a.M : 0);
        const int blocks = (int)std::min<long long>((total + 255) / 256, (long long)ctx->num_sms * 8);
        launch_step_kernel(ctx, ctx->compute, splitk_reduce_kernel, dim3((unsigned)blocks), dim3(256), 0, p);
        RST_TRY(after_launch(ctx, "splitk_reduce_kernel"));
    }
    return RST_OK;
}

// Tile configuration for problems with fewer than one wave of 128x128 tiles: 64x64
// tiles, 8 consumer warps (two per SM sub-partition, so that one warp's shared loads
// and barrier traffic hide behind the other's MMAs), 8 stages of 16 KiB (one CTA per
// SM has to keep enough bytes in flight to cover the latency of operands that are not
// in L2 yet; a TMA tile load takes about 1.5 us even from L2).
constexpr int kSmallBM = 64, kSmallBN = 64, kSmallWM = 2, kSmallWN = 4, kSmallStages = 8;
constexpr int kTinyB = 32;

// A few waves of large tiles with a mostly empty last one (512 tiles on 148 SMs: 3.46 waves,
// 13 % of the time on a quarter-full GPU): split K two to four ways when that fills the last
// wave to 95 % and leaves at least 32 k-tiles per split.
int large_tile_splits(const rst_ctx* ctx, long long tiles_large, long long k_tiles) {
    auto fill = [&](long long ctas) {
        const long long waves = (ctas + ctx->num_sms - 1) / ctx->num_sms;
        return (double)ctas / (double)(waves * ctx->num_sms);
    };
    if (tiles_large <= 4LL * ctx->num_sms && fill(tiles_large) < 0.95)
        for (int s = 2; s <= 4; ++s)
            if (k_tiles / s >= 32 && fill(tiles_large * s) >= 0.95) return s;
    return 1;
}

template <bool A_K, bool B_K>
int launch_layout(rst_ctx* ctx, const GemmArgs& a, GemmParams& p, bool* colsum_done) {
    const long long k_tiles = (a.K + kBK - 1) / kBK;
    const long long tiles_large = ((a.M + 127) / 128) * ((a.N + 127) / 128);
    if (tiles_large >= ctx->num_sms) {
        const int splits = large_tile_splits(ctx, tiles_large, k_tiles);
        if (!A_K && !B_K) {
            // the variant that also stores the transposed copy is an instantiation of its own, so
            // that the dW product keeps its registers
            if (p.Ct != nullptr) return launch_cfg<128, 128, 2, 4, 6, false, false, false, true>(ctx, a, p, splits);
        }
        return launch_cfg<128, 128, 2, 4, 6, A_K, B_K, false>(ctx, a, p, splits);
    }
    // Small problems: 64x64 tiles.  CTAs that share an SM share its f64 tensor pipe,
    // so more than one wave of CTAs buys nothing: split K only as far as the grid
    // still fits one wave, keeping at least two k-tiles per split and at most 64
    // splits (the reduce kernel reads every partial; measured on the batch-32 and
    // batch-4096 steps against 4/16: 2 % and 4 % faster).
    auto splits_for = [&](long long tiles) {
        long long splits = ctx->num_sms / tiles;
        splits = std::min(splits, k_tiles / 2);
        splits = std::min(splits, 64LL);
        if (k_tiles < 16) splits = 1;        // the reduce launch would cost more than the split saves
        return (int)std::max(splits, 1LL);
    };
    constexpr bool kFuse = !A_K && !B_K;     // the dW product also yields db
    if (kFuse && a.colsum_out && colsum_done) *colsum_done = true;
    // A product with at most 32 rows or columns (batch 32; the 10-class output layer) only
    // fills a quarter of a 64x64 tile, and on a dependent chain of such launches the time
    // of a k-tile is what counts: 32x32 tiles, one consumer warp per SM sub-partition,
    // finish a k-tile in a quarter of the tensor-pipe time.
    const long long tiles_tiny = ((a.M + kTinyB - 1) / kTinyB) * ((a.N + kTinyB - 1) / kTinyB);
    if ((a.M <= kTinyB || a.N <= kTinyB) && tiles_tiny <= ctx->num_sms)
        return launch_cfg<kTinyB, kTinyB, 2, 2, kSmallStages, A_K, B_K, kFuse>(ctx, a, p, splits_for(tiles_tiny));
    const long long tiles_small = ((a.M + kSmallBM - 1) / kSmallBM) * ((a.N + kSmallBN - 1) / kSmallBN);
    return launch_cfg<kSmallBM, kSmallBN, kSmallWM, kSmallWN, kSmallStages, A_K, B_K, kFuse>(ctx, a, p,
                                                                                              splits_for(tiles_small));
}

}  // namespace

bool gemm_writes_transposed(const rst_ctx* ctx, const GemmArgs& a) {
    if (a.a_kmajor || a.b_kmajor || !a.C_transposed) return false;
    if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.M > 0x7fffff00LL || a.N > 0x7fffff00LL || a.K > 0x7fffff00LL) return false;
    if ((a.M % 2) || (a.N % 4)) return false;
    if ((((uintptr_t)a.A | (uintptr_t)a.B | (uintptr_t)a.C_transposed) & 15u) != 0) return false;
    if ((((uintptr_t)a.C | (uintptr_t)a.mask_src | (uintptr_t)a.bias) & 31u) != 0) return false;
    if (a.epilogue != kEpiNone && a.epilogue != kEpiMask) return false;
    const long long tiles_large = ((a.M + 127) / 128) * ((a.N + 127) / 128);
    const long long k_tiles = (a.K + kBK - 1) / kBK;
    return tiles_large >= ctx->num_sms && large_tile_splits(ctx, tiles_large, k_tiles) == 1;
}

int launch_gemm(rst_ctx* ctx, const GemmArgs& a, bool* colsum_done) {
    if (colsum_done) *colsum_done = false;
    if (a.M == 0 || a.N == 0) return RST_OK;
    if (a.M > 0x7fffff00LL || a.N > 0x7fffff00LL || a.K > 0x7fffff00LL)
        return fail(ctx, RST_ERR_UNSUPPORTED, "GEMM extent beyond 2^31 (M %lld, N %lld, K %lld)", a.M, a.N, a.K);
    GemmParams p{};
    p.C = a.C; p.bias = a.bias; p.mask_src = a.mask_src; p.splitk_ws = nullptr;
    p.colsum_out = nullptr;
    p.status = ctx->d_status; p.divisor = a.divisor;
    p.wait_limit = a.wait_limit_cycles > 0 ? a.wait_limit_cycles : kWaitLimitCycles;
    p.starve = a.starve_producer ? 1 : 0;
    p.M = a.M; p.N = a.N; p.K = a.K; p.epilogue = a.epilogue; p.splits = 1;
    if (a.C_transposed) {
        if (!gemm_writes_transposed(ctx, a))
            return fail(ctx, RST_ERR_UNSUPPORTED, "a transposed copy of C is not available for this product");
        p.Ct = a.C_transposed;
    }

    // TMA needs 16-byte aligned bases and row pitches: the contiguous extent of
    // each operand must be even.
    const long long a_inner = a.a_kmajor ? a.K : a.M;
    const long long b_inner = a.b_kmajor ? a.K : a.N;
    const bool tma_ok = a.K > 0 && (a_inner % 2 == 0) && (b_inner % 2 == 0) &&
                        (((uintptr_t)a.A | (uintptr_t)a.B) & 15u) == 0;
    if (!tma_ok) {
        long long sam = a.a_kmajor ? a.K : 1, sak = a.a_kmajor ? 1 : a.M;
        long long sbk = a.b_kmajor ? 1 : a.N, sbn = a.b_kmajor ? a.K : 1;
        long long total = a.M * a.N;
        int blocks = (int)std::min<long long>((total + 255) / 256, (long long)ctx->num_sms * 8);
        gemm_f64_plain<<<blocks, 256, 0, ctx->compute>>>(a.A, a.B, sam, sak, sbk, sbn, p);
        return after_launch(ctx, "gemm_f64_plain");
    }
    if (a.a_kmajor && a.b_kmajor) return launch_layout<true, true>(ctx, a, p, colsum_done);
    if (a.a_kmajor && !a.b_kmajor) return launch_layout<true, false>(ctx, a, p, colsum_done);
    if (!a.a_kmajor && !a.b_kmajor) return launch_layout<false, false>(ctx, a, p, colsum_done);
    return fail(ctx, RST_ERR_UNSUPPORTED, "M-major A with K-major B is not implemented");
}

// The dW = dYᵀ·X / n products (with their db) of up to kMaxGroup layers in one launch plus
// one reduce launch.  Taken only when every product is in the small-tile regime and all
// their tiles fit one wave together; *grouped tells the caller whether it was (if not,
// nothing was launched and the caller issues the products one by one).
int launch_gemm_group(rst_ctx* ctx, const GemmArgs* args, int n, bool* grouped) {
    *grouped = false;
    if (n < 2 || n > kMaxGroup) return RST_OK;
    using C_ = Cfg<kSmallBM, kSmallBN, kSmallWM, kSmallWN, kSmallStages, false, false>;
    long long tiles_total = 0, units_total = 0;      // unit = one k-tile of one output tile
    for (int i = 0; i < n; ++i) {
        const GemmArgs& a = args[i];
        if (a.a_kmajor || a.b_kmajor || a.M <= 0 || a.N <= 0 || a.K <= 0) return RST_OK;
        if (a.M > 0x7fffff00LL || a.N > 0x7fffff00LL || a.K > 0x7fffff00LL) return RST_OK;
        if ((a.M % 2) || (a.N % 2) || ((((uintptr_t)a.A | (uintptr_t)a.B) & 15u) != 0)) return RST_OK;
        if (((a.M + 127) / 128) * ((a.N + 127) / 128) >= ctx->num_sms) return RST_OK;
        const long long tiles = ((a.M + kSmallBM - 1) / kSmallBM) * ((a.N + kSmallBN - 1) / kSmallBN);
        tiles_total += tiles;
        units_total += tiles * ((a.K + kBK - 1) / kBK);
    }
    if (tiles_total > ctx->num_sms) return RST_OK;

    // Smallest number of k-tiles per CTA for which all CTAs still fit one wave: CTAs that
    // share an SM share its tensor pipe, so a second wave would only add its fixed costs.
    auto ctas_for = [&](long long per_cta) {
        long long ctas = 0;
        for (int i = 0; i < n; ++i) {
            const long long tiles = ((args[i].M + kSmallBM - 1) / kSmallBM) * ((args[i].N + kSmallBN - 1) / kSmallBN);
            const long long kt = (args[i].K + kBK - 1) / kBK;
            ctas += tiles * ((kt + per_cta - 1) / per_cta);
        }
        return ctas;
    };
    long long per_cta = std::max(2LL, (units_total + ctx->num_sms - 1) / ctx->num_sms);
    while (ctas_for(per_cta) > ctx->num_sms) ++per_cta;

    GroupMaps maps;
    GroupParams gp{};
    gp.count = n;
    size_t ws_elems = 0, ws_offset[kMaxGroup] = {};
    long long reduce_elems = 0;
    // longest CTAs first: products in decreasing k-tiles per CTA
    int order[kMaxGroup];
    for (int i = 0; i < n; ++i) order[i] = i;
    auto kt_per_cta = [&](int i) {
        const long long kt = (args[i].K + kBK - 1) / kBK;
        const long long splits = (kt + per_cta - 1) / per_cta;
        return (kt + splits - 1) / splits;
    };
    std::stable_sort(order, order + n, [&](int x, int y) { return kt_per_cta(x) > kt_per_cta(y); });
    int cta = 0;
    for (int slot = 0; slot < n; ++slot) {
        const GemmArgs& a = args[order[slot]];
        GemmParams& p = gp.p[slot];
        p.C = a.C; p.bias = a.bias; p.mask_src = a.mask_src; p.colsum_out = a.colsum_out;
        p.status = ctx->d_status; p.divisor = a.divisor;
        p.wait_limit = kWaitLimitCycles;
        p.M = a.M; p.N = a.N; p.K = a.K; p.epilogue = a.epilogue;
        p.tiles_m = (int)((a.M + kSmallBM - 1) / kSmallBM);
        p.tiles_n = (int)((a.N + kSmallBN - 1) / kSmallBN);
        p.k_tiles = (int)((a.K + kBK - 1) / kBK);
        const int want = (int)((p.k_tiles + per_cta - 1) / per_cta);
        p.k_tiles_per_split = (p.k_tiles + want - 1) / want;
        p.splits = (p.k_tiles + p.k_tiles_per_split - 1) / p.k_tiles_per_split;
        RST_TRY(encode_map(ctx, &maps.a[slot], a.A, a.M, a.K, 16, kBK));
        RST_TRY(encode_map(ctx, &maps.b[slot], a.B, a.N, a.K, 16, kBK));
        gp.first_cta[slot] = cta;
        cta += p.tiles_m * p.tiles_n * p.splits;
        if (p.splits > 1) {
            ws_offset[slot] = ws_elems;                              // the base is added once it is known
            ws_elems += (size_t)p.splits * ((size_t)a.M * (size_t)a.N + (size_t)a.M);
            ws_elems = (ws_elems + 1) & ~(size_t)1;                  // keep every region 16-byte aligned
            reduce_elems = std::max(reduce_elems, (long long)(a.M * a.N + (a.colsum_out ? a.M : 0)));
        }
    }
    for (int slot = n; slot <= kMaxGroup; ++slot) gp.first_cta[slot] = cta;
    if (ws_elems) {
        RST_TRY(ensure_scratch(ctx, (void**)&ctx->splitk_ws, &ctx->splitk_ws_bytes, ws_elems * sizeof(double),
                               "split-K"));
        for (int slot = 0; slot < n; ++slot)
            if (gp.p[slot].splits > 1) gp.p[slot].splitk_ws = ctx->splitk_ws + ws_offset[slot];
    }

    auto kernel = gemm_f64_tma_dmma_grouped<kSmallBM, kSmallBN, kSmallWM, kSmallWN, kSmallStages, false, false, true>;
    RST_TRY(allow_dynamic_smem(ctx, reinterpret_cast<const void*>(kernel), C_::kSmemBytes));
    launch_step_kernel(ctx, ctx->compute, kernel, dim3((unsigned)cta), dim3(C_::kThreads), (size_t)C_::kSmemBytes,
                       maps, gp);
    RST_TRY(after_launch(ctx, "gemm_f64_tma_dmma_grouped"));
    if (reduce_elems) {
        const int blocks = (int)std::min<long long>((reduce_elems + 255) / 256, (long long)ctx->num_sms * 8);
        launch_step_kernel(ctx, ctx->compute, splitk_reduce_grouped_kernel, dim3((unsigned)blocks), dim3(256), 0, gp);
        RST_TRY(after_launch(ctx, "splitk_reduce_grouped_kernel"));
    }
    *grouped = true;
    return RST_OK;
}

}  // namespace rst
