// Implicit-GEMM convolution on the 5th-generation tensor cores (sm_100a).
//
// GEMM view: M = output pixels, N = output channels, K = kh*kw*Cin.  No im2col buffer exists:
// for every kernel tap (r,s) and channel block the A operand is a TMA tiled load of a shifted
// TW x TH x TN box of NHWC pixels (out-of-bounds rows and columns are zero-filled by the TMA
// unit, which is the convolution's zero padding), landing in shared memory as 128 K-major rows
// in the hardware swizzle; the B operand is a TMA load of the packed weight matrix
// [Cout][kh][kw][Cin].  Stride-2 layers read one of four "parity" views of the input (every
// second row / column, offset by 0 or 1) so that a box is still a dense rectangle.
//
// Persistent CTAs: two per SM with 10 warps each for N tiles of up to 128 channels, one per SM with
// 18 warps for wider ones.
//   warp 0   TMA producer (lane g issues K block g of a stage) - fills a ring of shared-memory stages
//   warp 1   MMA issuer (one lane) + TMEM owner                 - tcgen05.mma, fp32 / int32 accumulators
//                                                                 in as many TMEM buffers as fit (2-4)
//   warps 2+ epilogue, in groups of four warps (one per TMEM     - tile i uses buffer i % buffers and
//            lane quarter)                                        group i % groups
//
// Main loops: the tap loop above; the row-box loop for stride-1 layers (one box of TW + kw - 1 pixels per kernel
// row, the kw taps read through descriptors that start 0, 1, .. pixels into the swizzled box); CTA pairs for wide
// tiles (two CTAs of a cluster share every MMA, tcgen05 cta_group::2, and each loads half of the weight rows).
// What bounds this kernel are its serial roles - one producing and one issuing thread per CTA, epilogue warps
// whose own instruction streams stall - and, for narrow N tiles, the shared-memory reads of the tensor pipe; every
// loop of a single-thread role is therefore table-driven, unrolled and free of divisions.  Two epilogues exist:
//   quad  (N tile a multiple of 32 channels): accumulators leave TMEM in the 16x256b shape, in which four
//         neighbouring lanes hold one pixel; the B operand is loaded through a tensor map that permutes the
//         output channels inside each 32-channel block so that those four lanes hold channels 0-7, 8-15,
//         16-23, 24-31 of the pixel.  Residual loads and output stores of a warp then cover 8 pixels x 64
//         contiguous bytes (whole 32-byte sectors) instead of 32 separate pieces.
//   row   (any N tile, ragged channel counts): a thread owns one pixel (one TMEM lane) and walks its
//         channels 16 at a time (32 at a time, with whole-sector stores, when the only output is int8).
// Variants with their own instantiation: patch mode for few-channel stride-2 stems (the raw input patch
// read through un-swizzled overlapping descriptors) with a 3x3/2 max pooling in the epilogue, and the
// per-channel PReLU activation.
// All mbarrier waits are bounded; when one runs out the kernel raises the context's error
// word, every role leaves its loop, TMEM is freed and the launch returns normally.
#include "conv_common.cuh"
#include "ptx_sm100.cuh"

#include <cudaTypedefs.h>

#include <mutex>
#include <set>
#include <utility>

namespace exb {
namespace {

constexpr int kMaxStages = 8;
constexpr int kFirstEpiWarp = 2;   // warp 0 producer, warp 1 MMA issuer, epilogue warps from here on
constexpr int kMaxAccBufs = 4;
constexpr int kConstCh = 64;      // output channels of the pool epilogue (scale / bias travel as launch parameters)
constexpr int kTileM = 128;
constexpr uint32_t kMaxSpins = 1u << 21;  // tens of milliseconds at least; a legitimate wait is microseconds

enum EpiKind { kEpiRow = 0, kEpiQuad = 1, kEpiPool = 2 };

struct ConvTcParams {
    CUtensorMap tmA[4];
    CUtensorMap tmB;
    int N, OH, OW;
    int TW, TH, TN;
    int tiles_w, tiles_h, tiles_nb;  // M tiles per dimension
    int n_tiles;                     // N (cout) tiles
    int BN;
    int kh, kw, stride, pad_t, pad_l;
    int cin_pad;      // channels per tap in the packed weights (= physical input channels)
    int cblks;        // K blocks per tap
    int kb_elems;     // channels per K block
    int kb_bytes;     // 32 / 64 / 128
    int stages;
    int a_bytes, b_bytes;   // shared-memory bytes per stage
    int a_tx_bytes;         // bytes one A box delivers
    int tmem_cols;
    int acc_bufs;     // accumulator buffers in TMEM (2 or 4)
    int epi_groups;   // epilogue warp groups (2 or 4); group g drains tiles g, g + epi_groups, ... of the CTA
    int cout_pad;     // entries of the scale / bias arrays
    uint32_t idesc;
    int has_res;
    EpiParams e;
    int* error;
    int kgroup;       // K blocks per pipeline stage (one mbarrier round trip per stage)
    int fold;         // folded K layout (see FoldPlan): one K block per kernel row
    int b_resident;   // the whole weight slice stays in shared memory for the life of the CTA
    int b_region;     // bytes of the B region in shared memory (ring or resident copy)
    int b_perm;       // tmB is the 5-D channel-permuting map of the quad epilogue
    int k_iters;      // K units per tile: (tap, channel block) pairs, or (kernel row, channel block) pairs in row-box mode
    // "Row-box" mode for stride-1 convolutions (TW = 8): one K unit is the TMA box of TW + kw - 1 pixels x TH x TN of
    // ONE kernel row and channel block; the kw taps of that row are the same box read through descriptors that start
    // 0, 1, .. kw-1 pixels in (an 8-row group of the tile = 8 consecutive pixels of a box row, the next group one
    // box row = a_sbo bytes on).  The hardware swizzle is a function of the shared-memory address, so a descriptor may
    // start anywhere in a swizzle atom; the tensor pipe reads such operands at full rate (exb_tensor_peak_probe_layout).
    // Every input byte then crosses from L2 into shared memory kh * (TW + kw - 1) / TW times instead of kh * kw times:
    // that traffic, not the tensor pipe, is what bounds the tap-by-tap loop.
    int rowbox;
    int taps;         // B blocks (taps) per K unit: kw in row-box mode, else 1
    int a_sbo;        // bytes between consecutive 8-row groups of the A operand
    // "Patch" mode for stride-2 stems on NHWC4 rows (8-byte pixels): the A operand of kernel row r
    // is the raw input patch itself, read through an un-swizzled descriptor whose rows are 16
    // bytes apart (= one output column) and whose K chunks are 16 bytes apart as well, so the
    // overlapping 8-pixel windows of neighbouring output columns are never duplicated in shared
    // memory: one TMA load of (2*TH + kh - 2) x 24 pixels per tile instead of kh boxes of
    // 128 x 64 bytes.
    int patch;
    int patch_rows;    // input rows per tile
    int patch_pitch;   // bytes per patch row in shared memory
    const void* w_global;   // packed weights (patch mode copies them into core-matrix layout)
    // Tile origins: first output column / row of tile index i is i * step + org (step = TW / TH and
    // org = 0 unless tiles overlap).
    int step_w, step_h, org;
    // Fused 3x3/2 pad-1 max pooling (patch mode, BN = 64): an 8 x 16 tile of the convolution output
    // starts at (6*tx - 1, 14*ty - 1), so it holds every input of the 3 x 7 pooled outputs that
    // start at (3*tx, 7*ty); neighbouring tiles overlap by two rows / columns, which are recomputed.
    int pool, PH, PW;
    // Pool epilogue: per-channel scale and bias as launch parameters.  Its channel offsets are compile-time constants,
    // so the values become constant-bank operands of the FMAs: no load instruction and no traffic on the load/store
    // pipe, where a shared-memory load at an address common to the warp costs one wavefront per four bytes.  (With
    // run-time offsets - the other epilogues - a constant-bank load per value measured slower than the shared-memory
    // copy.)
    alignas(16) float c_scale[kConstCh];
    alignas(16) float c_bias[kConstCh];
};

struct TileCoord {
    int ow0, oh0, n0, ntile;
};

// Walks the tile sequence first, first + step, first + 2 * step, ... of one role without a division per tile: the
// position is kept as mixed-radix digits (N tile, tile column, tile row, image group) and the step, split into the
// same digits once, is added with carries.  (Every role is a single thread or a warp whose instructions depend on
// one another; three integer divisions per tile were a visible part of the tile period of short-K layers.)
struct TileCursor {
    int nt, w, h, n;        // position
    int dnt, dw, dh, dn;    // step
    __device__ __forceinline__ TileCursor(const ConvTcParams& p, int first, int step) {
        nt = first % p.n_tiles;
        int m = first / p.n_tiles;
        w = m % p.tiles_w;
        m /= p.tiles_w;
        h = m % p.tiles_h;
        n = m / p.tiles_h;
        dnt = step % p.n_tiles;
        m = step / p.n_tiles;
        dw = m % p.tiles_w;
        m /= p.tiles_w;
        dh = m % p.tiles_h;
        dn = m / p.tiles_h;
    }
    __device__ __forceinline__ void advance(const ConvTcParams& p) {
        nt += dnt;
        int c = nt >= p.n_tiles;
        if (c) nt -= p.n_tiles;
        w += dw + c;
        c = w >= p.tiles_w;
        if (c) w -= p.tiles_w;
        h += dh + c;
        c = h >= p.tiles_h;
        if (c) h -= p.tiles_h;
        n += dn + c;
    }
    __device__ __forceinline__ TileCoord coord(const ConvTcParams& p) const {
        TileCoord c;
        c.ntile = nt;
        c.ow0 = w * p.step_w + p.org;
        c.oh0 = h * p.step_h + p.org;
        c.n0 = n * p.TN;
        return c;
    }
};

// One pixel's 16 consecutive channels starting at channel `cl`: v = acc * scale + bias (+ residual) -> activation ->
// first / second output.  `pix` is the pixel's index in the output tensor.  The accumulators are raw[kStep * (i / 2) +
// kFirst + (i & 1)], i = 0..15: (16, 2, 0) reads a plain 16-register chunk, (32, 4, 0) / (32, 4, 2) the first / second
// pixel of a 16x256b fragment.
template <bool kInt8, bool kPrelu, int kRegs, int kStep, int kFirst>
__device__ __forceinline__ void epi_row16(const EpiParams& e, const float4 (&sc)[4], const float4 (&bi)[4], int cl, int64_t pix,
                                          bool add_res, const uint32_t (&res)[8], const uint32_t (&raw)[kRegs]) {
    float v[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 s4 = sc[i], b4 = bi[i];
        v[4 * i + 0] = epi_value<kInt8>(raw[kStep * (2 * i) + kFirst], s4.x, b4.x);
        v[4 * i + 1] = epi_value<kInt8>(raw[kStep * (2 * i) + kFirst + 1], s4.y, b4.y);
        v[4 * i + 2] = epi_value<kInt8>(raw[kStep * (2 * i + 1) + kFirst], s4.z, b4.z);
        v[4 * i + 3] = epi_value<kInt8>(raw[kStep * (2 * i + 1) + kFirst + 1], s4.w, b4.w);
    }
    if (add_res) {
        const __half2* h = reinterpret_cast<const __half2*>(res);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float2 f = __half22float2(h[i]);
            v[2 * i] += f.x;
            v[2 * i + 1] += f.y;
        }
    }
    if constexpr (kPrelu) prelu_vec16(v, e.slope + cl);
    else act_vec16(v, e.act);
    const int64_t off = pix * e.y_pitch + cl;
    uint32_t acc[16];       // raw accumulators in channel order (only the int32 output reads them)
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = raw[kStep * (i >> 1) + kFirst + (i & 1)];
    epi_store_vec16(e.y, e.out_dtype, off, v, e.out_scale, acc);
    if (e.out2_dtype >= 0) epi_store_vec16(e.y2, e.out2_dtype, off, v, e.out2_scale, acc);
}

// Two pixels' 8 consecutive channels from one 16x256b.x4 fragment (raw[4g + e] first pixel, raw[4g + 2 + e] second
// pixel, channels cl + 2g + e).  Scale and bias are read once for both pixels, from the quad-ordered copy: the four
// floats of channels 8*j + 4*i .. + 3 of a 32-channel block sit at 32*block + 16*i + 4*j, so that the four lanes of a
// pixel read one contiguous 64-byte piece per load (channel order would put neighbouring lanes on the same banks).
template <bool kInt8, bool kPrelu>
__device__ __forceinline__ void epi_quad_rows(const EpiParams& e, const float* q_scale, const float* q_bias, int cl, int cq,
                                              int pa, int pb, bool add_res, const uint4& ra, const uint4& rb,
                                              const uint32_t (&raw)[16]) {
    float va[8], vb[8];
    const float4* sc = reinterpret_cast<const float4*>(q_scale + (cl & ~31) + 4 * cq);
    const float4* bi = reinterpret_cast<const float4*>(q_bias + (cl & ~31) + 4 * cq);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float4 s4 = sc[4 * i], b4 = bi[4 * i];
        va[4 * i + 0] = epi_value<kInt8>(raw[8 * i + 0], s4.x, b4.x);
        va[4 * i + 1] = epi_value<kInt8>(raw[8 * i + 1], s4.y, b4.y);
        va[4 * i + 2] = epi_value<kInt8>(raw[8 * i + 4], s4.z, b4.z);
        va[4 * i + 3] = epi_value<kInt8>(raw[8 * i + 5], s4.w, b4.w);
        vb[4 * i + 0] = epi_value<kInt8>(raw[8 * i + 2], s4.x, b4.x);
        vb[4 * i + 1] = epi_value<kInt8>(raw[8 * i + 3], s4.y, b4.y);
        vb[4 * i + 2] = epi_value<kInt8>(raw[8 * i + 6], s4.z, b4.z);
        vb[4 * i + 3] = epi_value<kInt8>(raw[8 * i + 7], s4.w, b4.w);
    }
    if (add_res) {
        const __half2* ha = reinterpret_cast<const __half2*>(&ra);
        const __half2* hb = reinterpret_cast<const __half2*>(&rb);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 fa = __half22float2(ha[i]), fb = __half22float2(hb[i]);
            va[2 * i] += fa.x;
            va[2 * i + 1] += fa.y;
            vb[2 * i] += fb.x;
            vb[2 * i + 1] += fb.y;
        }
    }
    if constexpr (kPrelu) {
        const float4 l0 = __ldg(reinterpret_cast<const float4*>(e.slope + cl)), l1 = __ldg(reinterpret_cast<const float4*>(e.slope + cl) + 1);
        const float sl[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            va[i] = va[i] >= 0.f ? va[i] : va[i] * sl[i];
            vb[i] = vb[i] >= 0.f ? vb[i] : vb[i] * sl[i];
        }
    } else {
        apply_act_vec(va, e.act);
        apply_act_vec(vb, e.act);
    }
    if (pa >= 0) {
        const int64_t off = (int64_t)pa * e.y_pitch + cl;
        epi_store_vec8(e.y, e.out_dtype, off, va, e.out_scale);
        if (e.out2_dtype >= 0) epi_store_vec8(e.y2, e.out2_dtype, off, va, e.out2_scale);
    }
    if (pb >= 0) {
        const int64_t off = (int64_t)pb * e.y_pitch + cl;
        epi_store_vec8(e.y, e.out_dtype, off, vb, e.out_scale);
        if (e.out2_dtype >= 0) epi_store_vec8(e.y2, e.out2_dtype, off, vb, e.out2_scale);
    }
}

// The MMAs of one row-box unit, fully unrolled: tap s reads the box s pixels further in (kSteps 32-byte K steps per
// pixel) against the weight block of that tap.  The issuing thread retires one instruction every few cycles, so
// every address computed at run time shows in the MMA rate of narrow tiles.
template <bool kInt8, int kTaps, int kSteps, bool kPair>
__device__ __forceinline__ void rowbox_unit(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                            uint32_t idesc, uint32_t b_tap, uint32_t accumulate) {
#pragma unroll
    for (int sx = 0; sx < kTaps; ++sx) {
#pragma unroll
        for (int ks = 0; ks < kSteps; ++ks) {
            if (kPair)
                ptx::tc_mma_ab_pair<kInt8>(d_tmem, a_lo + (uint32_t)(sx * 2 * kSteps + 2 * ks), a_hi, b_lo + (uint32_t)(2 * ks), b_hi,
                                           idesc, (sx | ks) ? 1u : accumulate);
            else
                ptx::tc_mma_ab<kInt8>(d_tmem, a_lo + (uint32_t)(sx * 2 * kSteps + 2 * ks), a_hi, b_lo + (uint32_t)(2 * ks), b_hi, idesc,
                                      (sx | ks) ? 1u : accumulate);
        }
        b_lo += b_tap;
    }
}

// kEpiWarps = 16: one CTA per SM (all of shared memory and TMEM, 2-4 accumulator buffers).
// kEpiWarps = 8:  two CTAs per SM for layers with narrow N tiles: two MMA issuers and two producers per SM;
//                 each CTA takes half the shared memory and at most 256 TMEM columns.
// kEpi: which epilogue (see the head of the file); each is its own instantiation so that the others keep
// their register allocation.  kPrelu: the activation is the per-channel PReLU.
// kPair: the CTA is one of a cluster of two that share every MMA (tcgen05 cta_group::2, M = 256): each CTA loads
//        the A box of its own M tile and HALF of the N tile's weight rows, the rank-0 CTA's thread issues the MMAs
//        for both, each CTA drains its own 128 accumulator rows.  Halves the weight stream per SM (wide layers).
template <bool kInt8, int kEpiWarps, int kEpi, bool kPrelu = false, bool kPair = false>
__global__ void __launch_bounds__((kFirstEpiWarp + kEpiWarps) * 32, kEpiWarps == 8 ? 2 : 1)
    conv_tc_kernel(const __grid_constant__ ConvTcParams p) {
    constexpr int kThreads = (kFirstEpiWarp + kEpiWarps) * 32;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kMaxStages];
    __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
    __shared__ __align__(8) uint64_t tfull_bar[kMaxAccBufs];
    __shared__ __align__(8) uint64_t tempty_bar[kMaxAccBufs];
    __shared__ __align__(8) uint64_t bres_bar;
    __shared__ uint32_t tmem_base_smem;
    __shared__ int abort_flag;
    __shared__ int pool_fail[kMaxAccBufs];

    // Operand ring, 1024-byte aligned (the widest swizzle atom).
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + (size_t)p.stages * p.kgroup * p.a_bytes;
    // Per-output-channel scale and bias of every N tile, staged once per CTA.
    float* s_scale = reinterpret_cast<float*>(smem_b + (size_t)p.b_region);
    float* s_bias = s_scale + p.n_tiles * p.BN;
    // Per K iteration (tap, channel block): TMA coordinates that do not depend on the tile.
    int4* k_tab = reinterpret_cast<int4*>(s_bias + p.n_tiles * p.BN);
    // Pool mode: one 128-pixel x 64-channel fp16 staging tile per epilogue group.
    uint8_t* pool_stage = reinterpret_cast<uint8_t*>(k_tab + p.k_iters);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // Units of work: tiles, or (pair mode) pairs of tiles that are neighbours along the image-group dimension; unit u
    // of a pair is tile (.., 2 * q + rank).  first_unit / unit_step: this CTA's (cluster's) share of the sequence.
    const uint32_t cta_rank = kPair ? ptx::cluster_ctarank() : 0u;
    const int total_tiles = p.tiles_w * p.tiles_h * (kPair ? (p.tiles_nb + 1) / 2 : p.tiles_nb) * p.n_tiles;
    const int first_unit = kPair ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int unit_step = kPair ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    auto tile_of = [&](const TileCursor& c) -> TileCoord {
        TileCoord tc = c.coord(p);
        if (kPair) tc.n0 = (2 * c.n + (int)cta_rank) * p.TN;
        return tc;
    };
    const int k_iters = p.k_iters;

    // Let the next kernel of the stream be scheduled as soon as SMs free up (it waits for this
    // grid's completion at its own griddepcontrol.wait before it reads or writes global memory).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int i = 0; i < kMaxAccBufs; ++i) pool_fail[i] = 0;
        for (int s = 0; s < p.stages; ++s) {
            ptx::mbar_init(&full_bar[s], 1);
            ptx::mbar_init(&empty_bar[s], 1);
        }
        for (int i = 0; i < p.acc_bufs; ++i) {
            ptx::mbar_init(&tfull_bar[i], 1);
            ptx::mbar_init(&tempty_bar[i], (kPair ? 2 : 1) * (kEpiWarps / p.epi_groups));   // pair: both CTAs' warps arrive at rank 0
        }
        ptx::mbar_init(&bres_bar, 1);
        ptx::fence_mbar_init();
        ptx::tma_prefetch_desc(&p.tmA[0]);
        ptx::tma_prefetch_desc(&p.tmB);
    }
    if (warp == 1) {
        if (kPair) {
            ptx::tmem_alloc_pair(&tmem_base_smem, (uint32_t)p.tmem_cols);
            ptx::tmem_relinquish_pair();
        } else {
            ptx::tmem_alloc(&tmem_base_smem, (uint32_t)p.tmem_cols);
            ptx::tmem_relinquish();
        }
    }
    for (int it = threadIdx.x; it < k_iters; it += kThreads) {
        if (p.fold) {   // one K block per kernel row: the box starts at the output column itself
            const int oh_ = it - p.pad_t;
            const int ph = p.stride == 2 ? (oh_ & 1) : 0;
            k_tab[it] = make_int4(0, 0, p.stride == 2 ? ((oh_ - ph) >> 1) : oh_, (it * p.kb_elems) | ((ph * 2) << 28));
            continue;
        }
        if (p.rowbox) {  // one unit per (kernel row, channel block): the box starts pad_l pixels left of the tile
            const int r = it / p.cblks, cb = it - r * p.cblks;
            k_tab[it] = make_int4(cb * p.kb_elems, -p.pad_l, r - p.pad_t, r * p.kw * p.cin_pad + cb * p.kb_elems);
            continue;
        }
        const int tap = it / p.cblks, cb = it - tap * p.cblks;
        const int r = tap / p.kw, sx = tap - r * p.kw;
        int view = 0, dw, dh;
        if (p.stride == 1) {
            dw = sx - p.pad_l;
            dh = r - p.pad_t;
        } else {
            const int ow_ = sx - p.pad_l, oh_ = r - p.pad_t;
            const int pw = ow_ & 1, ph = oh_ & 1;
            dw = (ow_ - pw) >> 1;
            dh = (oh_ - ph) >> 1;
            view = ph * 2 + pw;
        }
        k_tab[it] = make_int4(cb * p.kb_elems, dw, dh, (tap * p.cin_pad + cb * p.kb_elems) | (view << 28));
    }
    if (p.patch) {
        // Weights into the un-swizzled canonical K-major layout: for kernel row r, 16-byte K
        // chunk j, output channel n: r*(BN*64) + j*(BN*16) + (n/8)*128 + (n%8)*16.
        const uint4* src = static_cast<const uint4*>(p.w_global);
        const int total = p.kh * p.BN * 4;
        for (int i = threadIdx.x; i < total; i += kThreads) {
            const int j = i & 3, n = (i >> 2) % p.BN, r = (i >> 2) / p.BN;
            const uint4 v = n < p.cout_pad ? src[((size_t)n * p.kh + r) * 4 + j] : make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(smem_b + r * (p.BN * 64) + j * (p.BN * 16) + (n >> 3) * 128 + (n & 7) * 16) = v;
        }
        ptx::fence_proxy_async();   // generic-proxy writes, read by the tensor core through the async proxy
    }
    for (int c = threadIdx.x; c < p.n_tiles * p.BN; c += kThreads) {
        const bool in = c < p.cout_pad;
        // quad epilogue: channel 32*b + 8*j + 4*i + k is kept at 32*b + 16*i + 4*j + k (see epi_quad_rows)
        const int at = kEpi == kEpiQuad ? ((c & ~31) | ((c & 4) << 2) | ((c & 24) >> 1) | (c & 3)) : c;
        s_scale[at] = in ? p.e.scale[c] : 0.f;
        s_bias[at] = in ? p.e.bias[c] : 0.f;
    }
    // Programmatic dependent launch: everything above touches only this launch's own parameters,
    // constant weights and on-chip state, so it may run while the previous kernel of the stream is
    // still draining; nothing below may start before that kernel's memory is complete and visible.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (kPair) ptx::cluster_sync();      // the peer's barriers are initialised before anything signals them
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_smem;

    if (warp == 0) {
        // ------------------------------- TMA producer --------------------------------------
        // A pipeline stage holds `kgroup` K blocks.  Lane g issues the two loads of block g, so a
        // whole stage costs one pass through this loop body: a single thread retires only one
        // instruction every few cycles, which is what bounds small-K layers otherwise.
        const int G = p.kgroup;
        int stage = 0;
        uint32_t phase = 0;
        int ok = 1;
        const uint32_t a_base = ptx::smem_u32(smem_a) + (uint32_t)(lane * p.a_bytes);
        const uint32_t b_base = ptx::smem_u32(smem_b) + (uint32_t)(lane * p.taps * p.b_bytes);
        const uint32_t a_stage = (uint32_t)(G * p.a_bytes), b_stage = (uint32_t)(G * p.taps * p.b_bytes);
        const uint32_t full0 = ptx::smem_u32(&full_bar[0]), empty0 = ptx::smem_u32(&empty_bar[0]);
        const uint64_t mapA0 = reinterpret_cast<uint64_t>(&p.tmA[0]);
        const uint64_t mapB = reinterpret_cast<uint64_t>(&p.tmB);
        const bool bres = p.b_resident != 0;
        const bool bperm = p.b_perm != 0;
        const uint32_t tx = (uint32_t)(p.a_tx_bytes + (bres ? 0 : p.taps * p.b_bytes));
        if (bres && lane == 0) {
            // Weights stay resident: the slice [BN x K] is loaded once (n_tiles == 1 here), one block per tap and
            // channel block in tap-major order (row-box mode: unit (r, cb) holds taps (r, 0..kw-1)).
            // pair mode: each CTA keeps its half of the rows; both halves complete on the rank-0 CTA's barrier
            const uint32_t rb = kPair ? ptx::map_to_cta(ptx::smem_u32(&bres_bar), 0) : ptx::smem_u32(&bres_bar);
            if (!kPair || cta_rank == 0)
                ptx::mbar_arrive_expect_tx_u32(ptx::smem_u32(&bres_bar), (uint32_t)((kPair ? 2 : 1) * k_iters * p.taps * p.b_bytes));
            const int nrow = kPair ? (int)cta_rank * (p.BN >> 1) : 0;
            for (int it = 0; it < k_iters; ++it) {
                const int r = it / p.cblks, cb = it - r * p.cblks;
                for (int sx = 0; sx < p.taps; ++sx) {
                    const int blk = p.rowbox ? (r * p.kw + sx) * p.cblks + cb : it;
                    const uint32_t dst = ptx::smem_u32(smem_b) + (uint32_t)(blk * p.b_bytes);
                    const int kc = (k_tab[it].w & 0x0fffffff) + sx * p.cin_pad;
                    if (kPair) {
                        if (bperm) ptx::tma_load_5d_pair(dst, mapB, rb, kc, 0, 0, 0, nrow >> 5);
                        else ptx::tma_load_2d_pair(dst, mapB, rb, kc, nrow);
                    } else {
                        if (bperm) ptx::tma_load_5d_u32(dst, mapB, rb, kc, 0, 0, 0, 0);
                        else ptx::tma_load_2d_u32(dst, mapB, rb, kc, 0);
                    }
                }
            }
        }
        if (p.patch) {
            if (lane == 0) {
                const uint32_t bytes = (uint32_t)(p.patch_rows * p.patch_pitch);
                TileCursor cur(p, first_unit, unit_step);
                for (int t = first_unit; t < total_tiles && ok; t += unit_step, cur.advance(p)) {
                    const TileCoord tc = tile_of(cur);
                    // Fused pooling: patch ring and accumulator ring have the same length and tile i uses slot i % length
                    // of both, so the patch of a slot is free when the MMAs of the tile that used it have retired, which is
                    // what the slot's "accumulator full" barrier says - one commit per tile serves producer and epilogue
                    // (the issuing thread is what bounds that kernel).  The plain stem keeps its longer ring of patches.
                    if (!ptx::mbar_wait_bounded_u32((p.pool ? ptx::smem_u32(&tfull_bar[0]) : empty0) + stage * 8, phase ^ 1u, &abort_flag,
                                                    kMaxSpins)) {
                        ok = 0;
                        break;
                    }
                    const uint32_t fb = full0 + stage * 8;
                    ptx::mbar_arrive_expect_tx_u32(fb, bytes);
                    // x: first element of the window of output column ow0 (8 px wide, 4 left of
                    // 2*ow0 in image coordinates = 2*ow0 in padded coordinates), y: first input row
                    asm volatile(
                        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
                        " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(ptx::smem_u32(smem_a) + (uint32_t)(stage * p.a_bytes)),
                        "l"(mapA0), "r"(fb), "r"(tc.ow0 * 8), "r"(tc.oh0 * 2 - p.pad_t), "r"(tc.n0)
                        : "memory");
                    if (++stage == p.stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) {
                    atomicExch(p.error, 1);
                    for (int i = 0; i < 2000; ++i) __nanosleep(100);
                }
            }
        } else if (lane < G) {
            TileCursor cur(p, first_unit, unit_step);
            for (int t = first_unit; t < total_tiles && ok; t += unit_step, cur.advance(p)) {
                const TileCoord tc = tile_of(cur);
                // pair mode: this CTA loads its half of the N tile's weight rows
                const int ncoord = tc.ntile * p.BN + (kPair ? (int)cta_rank * (p.BN >> 1) : 0);
                for (int it0 = 0; it0 < k_iters; it0 += G) {
                    const int nb = min(G, k_iters - it0);
                    const bool mine = lane < nb;
                    int4 e = make_int4(0, 0, 0, 0);   // x: A channel coord, y: dw, z: dh, w: B k coord | view << 28
                    if (mine) e = k_tab[it0 + lane];
                    if (!ptx::mbar_wait_bounded_u32(empty0 + stage * 8, phase ^ 1u, &abort_flag, kMaxSpins)) {
                        ok = 0;
                        break;
                    }
                    if (kPair) {
                        // both CTAs' boxes complete on the rank-0 CTA's barrier, which expects the bytes of both
                        const uint32_t fb = ptx::map_to_cta(full0 + stage * 8, 0);
                        if (lane == 0 && cta_rank == 0) ptx::mbar_arrive_expect_tx_u32(full0 + stage * 8, 2u * tx * (uint32_t)nb);
                        if (mine) {
                            ptx::tma_load_4d_pair(a_base + stage * a_stage, mapA0 + ((uint32_t)e.w >> 28) * sizeof(CUtensorMap), fb,
                                                  e.x, tc.ow0 + e.y, tc.oh0 + e.z, tc.n0);
                            if (!bres) {
                                for (int sx = 0; sx < p.taps; ++sx) {
                                    const uint32_t dst = b_base + stage * b_stage + (uint32_t)(sx * p.b_bytes);
                                    const int kc = (e.w & 0x0fffffff) + sx * p.cin_pad;
                                    if (bperm) ptx::tma_load_5d_pair(dst, mapB, fb, kc, 0, 0, 0, ncoord >> 5);
                                    else ptx::tma_load_2d_pair(dst, mapB, fb, kc, ncoord);
                                }
                            }
                        }
                    } else {
                    const uint32_t fb = full0 + stage * 8;
                    if (lane == 0) ptx::mbar_arrive_expect_tx_u32(fb, tx * (uint32_t)nb);
                    if (mine) {
                        ptx::tma_load_4d_u32(a_base + stage * a_stage, mapA0 + ((uint32_t)e.w >> 28) * sizeof(CUtensorMap), fb,
                                             e.x, tc.ow0 + e.y, tc.oh0 + e.z, tc.n0);
                        if (!bres) {
                            for (int sx = 0; sx < p.taps; ++sx) {
                                const uint32_t dst = b_base + stage * b_stage + (uint32_t)(sx * p.b_bytes);
                                const int kc = (e.w & 0x0fffffff) + sx * p.cin_pad;
                                if (bperm) ptx::tma_load_5d_u32(dst, mapB, fb, kc, 0, 0, 0, ncoord >> 5);
                                else ptx::tma_load_2d_u32(dst, mapB, fb, kc, ncoord);
                            }
                        }
                    }
                    }
                    if (++stage == p.stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok) {
                if (lane == 0) atomicExch(p.error, 1);
                // Give copies already in flight time to land before this CTA's shared memory
                // can be handed to another CTA.
                for (int i = 0; i < 2000; ++i) __nanosleep(100);
            }
        }
    } else if (warp == 1) {
        // ------------------------------- MMA issuer ----------------------------------------
        if (lane == 0 && cta_rank == 0) {      // pair mode: the rank-0 CTA issues for both
            const int G = p.kgroup;
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            const int ksteps = p.kb_bytes / 32;
            const uint32_t full0 = ptx::smem_u32(&full_bar[0]), empty0 = ptx::smem_u32(&empty_bar[0]);
            const uint32_t tfull0 = ptx::smem_u32(&tfull_bar[0]), tempty0 = ptx::smem_u32(&tempty_bar[0]);
            // descriptor halves: low = (address >> 4) | LBO(=1) << 16, high = SBO | version | swizzle
            const uint64_t d0 = ptx::make_smem_desc(ptx::smem_u32(smem_a), (uint32_t)p.kb_bytes);
            const uint32_t desc_hi = (uint32_t)(d0 >> 32);
            const uint32_t a_lo0 = (uint32_t)d0;
            const uint32_t b_lo0 = (uint32_t)ptx::make_smem_desc(ptx::smem_u32(smem_b), (uint32_t)p.kb_bytes);
            const uint32_t a_blk = (uint32_t)p.a_bytes >> 4, b_blk = (uint32_t)p.b_bytes >> 4;
            const bool bres = p.b_resident != 0;
            const uint32_t a_stage = a_blk * G, b_stage = bres ? 0u : b_blk * G * p.taps;
            // row-box: A groups are a box row apart, tap s starts s pixels in; resident B blocks of one unit's taps
            // are cblks blocks apart (tap-major order), streamed ones follow each other
            const uint32_t a_hi = (desc_hi & ~0x3FFFu) | (((uint32_t)p.a_sbo >> 4) & 0x3FFFu);
            const uint32_t a_tap = (uint32_t)p.kb_bytes >> 4;
            const uint32_t b_tap = bres ? b_blk * p.cblks : b_blk;
            const uint32_t rb_row = (uint32_t)((p.kw - 1) * p.cblks) * b_blk;   // after a row's last channel block: skip its other taps
            const uint32_t idesc = p.idesc;
            if (bres && !ptx::mbar_wait_bounded(&bres_bar, 0, &abort_flag, kMaxSpins)) ok = false;
            for (int t = first_unit; t < total_tiles && ok; t += unit_step) {
                if (!ptx::mbar_wait_bounded_u32(tempty0 + acc * 8, acc_phase ^ 1u, &abort_flag, kMaxSpins)) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * p.BN);
                uint32_t accumulate = 0;
                uint32_t rb_b = b_lo0;
                int rb_cb = 0;
                if (p.patch) {
                    if (!ptx::mbar_wait_bounded_u32(full0 + stage * 8, phase, &abort_flag, kMaxSpins)) {
                        ok = false;
                        break;
                    }
                    // un-swizzled descriptors: A rows 16 B apart (LBO 16 B, SBO = two patch rows),
                    // B core matrices 128 B, K chunks BN*16 B apart
                    const uint32_t a0 = ((ptx::smem_u32(smem_a) + (uint32_t)(stage * p.a_bytes)) >> 4) | (1u << 16);
                    const uint32_t a_hi = ((uint32_t)(2 * p.patch_pitch) >> 4) | (1u << 14);
                    const uint32_t b0 = (ptx::smem_u32(smem_b) >> 4) | ((uint32_t)(p.BN * 16 >> 4) << 16);
                    const uint32_t b_hi = (128u >> 4) | (1u << 14);
                    for (int r = 0; r < p.kh; ++r) {
                        const uint32_t ar = a0 + (uint32_t)(r * p.patch_pitch >> 4);
                        const uint32_t br = b0 + (uint32_t)(r * p.BN * 64 >> 4);
#pragma unroll
                        for (int ks = 0; ks < 2; ++ks) {
                            asm volatile(
                                "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
                                "mov.b64 da, {%1, %2};\n\t"
                                "mov.b64 db, {%3, %4};\n\t"
                                "setp.ne.b32 p, %6, 0;\n\t"
                                "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
                                "r"(ar + ks * 2), "r"(a_hi), "r"(br + (uint32_t)(ks * 2 * (p.BN * 16 >> 4))), "r"(b_hi),
                                "r"(idesc), "r"(accumulate)
                                : "memory");
                            accumulate = 1;
                        }
                    }
                    if (!p.pool) ptx::tc_commit_u32(empty0 + stage * 8);
                    if (++stage == p.stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                } else
                for (int it0 = 0; it0 < k_iters; it0 += G) {
                    const int nb = min(G, k_iters - it0);
                    if (!ptx::mbar_wait_bounded_u32(full0 + stage * 8, phase, &abort_flag, kMaxSpins)) {
                        ok = false;
                        break;
                    }
                    uint32_t a_lo = a_lo0 + stage * a_stage;
                    uint32_t b_lo = b_lo0 + (bres ? (uint32_t)it0 * b_blk : stage * b_stage);
                    if (p.rowbox) {
                        for (int g = 0; g < nb; ++g) {
                            // resident weights: the unit's first block (tap-major order); streamed: the stage's
                            const uint32_t bu = bres ? rb_b : b_lo0 + stage * b_stage + (uint32_t)g * b_tap * p.taps;
                            if (p.taps == 3 && ksteps == 4) rowbox_unit<kInt8, 3, 4, kPair>(d_tmem, a_lo, a_hi, bu, desc_hi, idesc, b_tap, accumulate);
                            else if (p.taps == 3 && ksteps == 2) rowbox_unit<kInt8, 3, 2, kPair>(d_tmem, a_lo, a_hi, bu, desc_hi, idesc, b_tap, accumulate);
                            else
                                for (int sx = 0; sx < p.taps; ++sx)
                                    for (int ks = 0; ks < ksteps; ++ks)
                                        if (kPair)
                                            ptx::tc_mma_ab_pair<kInt8>(d_tmem, a_lo + sx * a_tap + 2 * ks, a_hi, bu + sx * b_tap + 2 * ks,
                                                                       desc_hi, idesc, (sx | ks) ? 1u : accumulate);
                                        else
                                        ptx::tc_mma_ab<kInt8>(d_tmem, a_lo + sx * a_tap + 2 * ks, a_hi, bu + sx * b_tap + 2 * ks, desc_hi,
                                                              idesc, (sx | ks) ? 1u : accumulate);
                            accumulate = 1;
                            a_lo += a_blk;
                            rb_b += b_blk;
                            if (++rb_cb == p.cblks) {
                                rb_cb = 0;
                                rb_b += rb_row;
                            }
                        }
                    } else
                    for (int g = 0; g < nb; ++g) {
                        if (kPair) {
                            if (ksteps == 4) {
                                ptx::tc_mma_lohi_pair<kInt8>(d_tmem, a_lo, b_lo, desc_hi, idesc, accumulate);
                                ptx::tc_mma_lohi_pair<kInt8>(d_tmem, a_lo + 2, b_lo + 2, desc_hi, idesc, 1);
                                ptx::tc_mma_lohi_pair<kInt8>(d_tmem, a_lo + 4, b_lo + 4, desc_hi, idesc, 1);
                                ptx::tc_mma_lohi_pair<kInt8>(d_tmem, a_lo + 6, b_lo + 6, desc_hi, idesc, 1);
                            } else {
                                for (int ks = 0; ks < ksteps; ++ks)
                                    ptx::tc_mma_lohi_pair<kInt8>(d_tmem, a_lo + 2 * ks, b_lo + 2 * ks, desc_hi, idesc, ks ? 1u : accumulate);
                            }
                        } else if (ksteps == 4) {
                            ptx::tc_mma_lohi<kInt8>(d_tmem, a_lo, b_lo, desc_hi, idesc, accumulate);
                            ptx::tc_mma_lohi<kInt8>(d_tmem, a_lo + 2, b_lo + 2, desc_hi, idesc, 1);
                            ptx::tc_mma_lohi<kInt8>(d_tmem, a_lo + 4, b_lo + 4, desc_hi, idesc, 1);
                            ptx::tc_mma_lohi<kInt8>(d_tmem, a_lo + 6, b_lo + 6, desc_hi, idesc, 1);
                        } else if (ksteps == 2) {
                            ptx::tc_mma_lohi<kInt8>(d_tmem, a_lo, b_lo, desc_hi, idesc, accumulate);
                            ptx::tc_mma_lohi<kInt8>(d_tmem, a_lo + 2, b_lo + 2, desc_hi, idesc, 1);
                        } else {
                            ptx::tc_mma_lohi<kInt8>(d_tmem, a_lo, b_lo, desc_hi, idesc, accumulate);
                        }
                        accumulate = 1;
                        a_lo += a_blk;
                        b_lo += b_blk;
                    }
                    // stage is free once these MMAs retire (pair mode: in both CTAs)
                    if (kPair) ptx::tc_commit_pair_u32(empty0 + stage * 8);
                    else ptx::tc_commit_u32(empty0 + stage * 8);
                    if (++stage == p.stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                // accumulator complete (pair mode: each CTA's epilogue drains its own 128 rows)
                if (kPair) ptx::tc_commit_pair_u32(tfull0 + acc * 8);
                else ptx::tc_commit_u32(tfull0 + acc * 8);
                if (++acc == p.acc_bufs) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
            if (!ok) atomicExch(p.error, 2);
        }
    } else if (warp >= kFirstEpiWarp) {
        // ------------------------------- epilogue ------------------------------------------
        // Tile i of this CTA's sequence is accumulated in buffer i % acc_bufs (use number i / acc_bufs of that
        // buffer gives the barrier parity) and drained by group i % epi_groups.  A group has kEpiWarps /
        // epi_groups warps: one or two per TMEM lane quarter; two share the quarter's work.
        const int e = warp - kFirstEpiWarp;
        const int q = warp & 3;                 // TMEM lane quarter: a warp can only reach lanes 32*(warp%4)..+31
        const int nsub = kEpiWarps / 4 / p.epi_groups;
        const int grp = (e >> 2) % p.epi_groups;
        const int sub = (e >> 2) / p.epi_groups;
        int ti = grp;
        bool ok = true;
        const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16);
        if constexpr (kEpi == kEpiPool) {
            // Convolution tile -> ReLU -> fp16 -> shared memory (16-byte units of a pixel row XOR-ed
            // with the row index so that neither phase has bank conflicts) -> 3x3/2 max -> global.
            // The group's four warps meet at a named barrier twice per tile; a warp whose bounded
            // wait ran out still arrives, and the whole group leaves together afterwards.
            const int row = q * 32 + lane;          // row of the M tile == TMEM lane
            const int tw = row % p.TW;
            const int th = (row / p.TW) % p.TH;
            uint8_t* stg = pool_stage + grp * (kTileM * 128);
            volatile int* failed = &pool_fail[grp];
            TileCursor cur(p, first_unit + grp * unit_step, p.epi_groups * unit_step);
            for (int t = first_unit + grp * unit_step; t < total_tiles; t += p.epi_groups * unit_step, ti += p.epi_groups, cur.advance(p)) {
                const TileCoord tc = tile_of(cur);
                const int ow = tc.ow0 + tw, oh = tc.oh0 + th;
                const bool inside = ow >= 0 && ow < p.OW && oh >= 0 && oh < p.OH;
                const int buf = ti % p.acc_bufs;
                const uint32_t acc_phase = (uint32_t)(ti / p.acc_bufs) & 1u;
                const uint32_t taddr = taddr0 + (uint32_t)(buf * p.BN);
                if (!ptx::mbar_wait_bounded_warp(&tfull_bar[buf], acc_phase, &abort_flag, kMaxSpins)) {
                    if (lane == 0) *failed = 1;
                } else {
                    ptx::tc_fence_after_sync();
                    // two loads of 32 channels; the activation (ReLU or ReLU6, checked by the host) is a clamp
                    const float act_hi = p.e.act == EXB_ACT_RELU6 ? 6.f : INFINITY;
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        uint32_t raw[32];
                        ptx::tmem_ld_32x32b_x32(taddr + half * 32, raw);
                        ptx::tmem_ld_wait();
                        uint32_t h[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            // compile-time offsets into the launch parameters: constant-bank operands of the FMAs
                            const int c = half * 32 + 2 * i;
                            const float v0 = fminf(fmaxf(epi_value<kInt8>(raw[2 * i], p.c_scale[c], p.c_bias[c]), 0.f), act_hi);
                            const float v1 = fminf(fmaxf(epi_value<kInt8>(raw[2 * i + 1], p.c_scale[c + 1], p.c_bias[c + 1]), 0.f), act_hi);
                            // positions outside the map never win: activated values are >= 0
                            const __half2 hv = inside ? __floats2half2_rn(v0, v1) : __floats2half2_rn(0.f, 0.f);
                            h[i] = *reinterpret_cast<const uint32_t*>(&hv);
                        }
                        uint8_t* dst = stg + row * 128;
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            *reinterpret_cast<uint4*>(dst + (((4 * half + u) ^ (row & 7)) << 4)) =
                                make_uint4(h[4 * u], h[4 * u + 1], h[4 * u + 2], h[4 * u + 3]);
                    }
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&tempty_bar[buf]);   // the accumulator is free again
                }
                if (grp == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
                else asm volatile("bar.sync 2, 128;" ::: "memory");
                if (*failed) {
                    ok = false;
                    break;
                }
                const int ph0 = (tc.oh0 + 1) >> 1, pw0 = (tc.ow0 + 1) >> 1;
                for (int item = row; item < 21 * 8; item += kTileM) {
                    const int pp = item >> 3, u = item & 7;
                    const int pr = pp / 3, pc = pp - 3 * pr;
                    const int ph = ph0 + pr, pw = pw0 + pc;
                    if (ph >= p.PH || pw >= p.PW) continue;
                    __half2 m[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) m[i] = __floats2half2_rn(0.f, 0.f);
#pragma unroll
                    for (int dr = 0; dr < 3; ++dr)
#pragma unroll
                        for (int dc = 0; dc < 3; ++dc) {
                            const int r = (2 * pr + dr) * 8 + 2 * pc + dc;
                            const uint4 tv = *reinterpret_cast<const uint4*>(stg + r * 128 + ((u ^ (r & 7)) << 4));
                            const __half2* th2 = reinterpret_cast<const __half2*>(&tv);
#pragma unroll
                            for (int i = 0; i < 4; ++i) m[i] = __hmax2(m[i], th2[i]);
                        }
                    const int64_t off = (((int64_t)tc.n0 * p.PH + ph) * p.PW + pw) * p.e.cout_stride + u * 8;
                    uint4 o;
                    o.x = *reinterpret_cast<const uint32_t*>(&m[0]);
                    o.y = *reinterpret_cast<const uint32_t*>(&m[1]);
                    o.z = *reinterpret_cast<const uint32_t*>(&m[2]);
                    o.w = *reinterpret_cast<const uint32_t*>(&m[3]);
                    *reinterpret_cast<uint4*>(static_cast<__half*>(p.e.y) + off) = o;
                    if (p.e.out2_dtype == EXB_I8) {
                        const float2 f0 = __half22float2(m[0]), f1 = __half22float2(m[1]);
                        const float2 f2 = __half22float2(m[2]), f3 = __half22float2(m[3]);
                        uint2 qv;
                        qv.x = quant_pack4(f0.x, f0.y, f1.x, f1.y, p.e.out2_scale);
                        qv.y = quant_pack4(f2.x, f2.y, f3.x, f3.y, p.e.out2_scale);
                        *reinterpret_cast<uint2*>(static_cast<int8_t*>(p.e.y2) + off) = qv;
                    }
                }
                // staging may be overwritten after this one
                if (grp == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
                else asm volatile("bar.sync 2, 128;" ::: "memory");
            }
        } else if constexpr (kEpi == kEpiQuad) {
            // Four neighbouring lanes hold one pixel: lane l of a 16-lane half covers tile rows r = l / 4 and
            // r + 8 and, of every 32-channel block, channels 8 * (l % 4) .. + 7 (the B tensor map stores
            // channel 8*j + 2*g + e of a block in accumulator column 8*g + 2*j + e, which is where the 16x256b
            // shape puts registers 4*g + e of lane quad member j).  A warp's 16-byte accesses therefore cover
            // 8 pixels x 64 contiguous bytes, every 32-byte sector whole.
            const int cq = lane & 3;
            const int nblk = p.BN >> 5;
            const int h_begin = nsub == 2 ? sub : 0, h_end = nsub == 2 ? sub + 1 : 2;
            // tile rows of this thread: [half][0 / +8], packed tw | th << 8 | tn << 16, bit 31 = row outside the box
            uint32_t rowpack[2][2];
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const int row = q * 32 + h * 16 + k * 8 + (lane >> 2);
                    const int tw = row % p.TW, th = (row / p.TW) % p.TH, tn = row / (p.TW * p.TH);
                    rowpack[h][k] = (uint32_t)tw | ((uint32_t)th << 8) | ((uint32_t)tn << 16) |
                                    (row < p.TW * p.TH * p.TN ? 0u : 0x80000000u);
                }
            // pixel index of a packed row in tile `c`, or -1 when the row lies outside the output
            auto pixel_of = [&](const TileCoord& c, uint32_t rp) -> int {
                const int ow = c.ow0 + (int)(rp & 0xff), oh = c.oh0 + (int)((rp >> 8) & 0xff);
                const int n = c.n0 + (int)((rp >> 16) & 0x7fff);
                if ((rp >> 31) || ow >= p.OW || oh >= p.OH || n >= p.N) return -1;
                return (n * p.OH + oh) * p.OW + ow;
            };
            const bool want_res = p.has_res != 0;
            TileCursor cur(p, first_unit + grp * unit_step, p.epi_groups * unit_step);
            for (int t = first_unit + grp * unit_step; t < total_tiles && ok; t += p.epi_groups * unit_step, ti += p.epi_groups) {
                const TileCoord tc = tile_of(cur);
                cur.advance(p);            // from here on: this group's next tile
                const int buf = ti % p.acc_bufs;
                const uint32_t acc_phase = (uint32_t)(ti / p.acc_bufs) & 1u;
                const int c0 = tc.ntile * p.BN + cq * 8;       // first channel of this thread in block 0
                // The residual lines of this group's NEXT tile are asked into L2 now (no register cost): when that
                // tile's turn comes its residual loads find them a few hundred cycles away instead of in DRAM.
                if (want_res && t + p.epi_groups * unit_step < total_tiles) {
                    const TileCoord c2 = tile_of(cur);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if (h < h_begin || h >= h_end) continue;
#pragma unroll
                        for (int k = 0; k < 2; ++k) {
                            const int px = pixel_of(c2, rowpack[h][k]);
                            if (px < 0) continue;
                            const __half* r2 = p.e.residual + (int64_t)px * p.e.cout_stride + c2.ntile * p.BN;
                            for (int l = cq; l * 64 < p.BN; l += 4)      // one 128-byte line per pixel and 64 channels
                                if (c2.ntile * p.BN + l * 64 < p.e.cout_stride) asm volatile("prefetch.global.L2 [%0];" ::"l"(r2 + l * 64));
                        }
                    }
                }
                // This thread's fragments of the tile: tile-row halves h_begin .. h_end - 1, nblk 32-channel blocks each,
                // fragment f = (half, block).  The residual of fragment f + 1 is requested before fragment f is
                // worked on, and that of the first fragment before the accumulator is even complete: a fragment's
                // arithmetic is a few hundred cycles, a residual load from L2 under load considerably more.
                const int pa0 = pixel_of(tc, h_begin ? rowpack[1][0] : rowpack[0][0]), pb0 = pixel_of(tc, h_begin ? rowpack[1][1] : rowpack[0][1]);
                const int pa1 = pixel_of(tc, rowpack[1][0]), pb1 = pixel_of(tc, rowpack[1][1]);
                const int nfrag = (h_end - h_begin) * nblk;
                auto res_load = [&](int f, uint4& a, uint4& b) {
                    a = make_uint4(0, 0, 0, 0);
                    b = make_uint4(0, 0, 0, 0);
                    const bool second = f >= nblk;
                    const int cl = c0 + (second ? f - nblk : f) * 32;
                    if (want_res && f < nfrag && cl < p.e.cout_stride) {
                        const int pa = second ? pa1 : pa0, pb = second ? pb1 : pb0;
                        if (pa >= 0) a = __ldg(reinterpret_cast<const uint4*>(p.e.residual + (int64_t)pa * p.e.cout_stride + cl));
                        if (pb >= 0) b = __ldg(reinterpret_cast<const uint4*>(p.e.residual + (int64_t)pb * p.e.cout_stride + cl));
                    }
                };
                uint4 ra, rb;
                res_load(0, ra, rb);
                if (!ptx::mbar_wait_bounded_warp(&tfull_bar[buf], acc_phase, &abort_flag, kMaxSpins)) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
#pragma unroll 1
                for (int f = 0; f < nfrag; ++f) {
                    const bool second = f >= nblk;
                    const int b = second ? f - nblk : f;
                    const int h = second ? 1 : h_begin;
                    const int cl = c0 + b * 32;
                    uint4 na, nb;
                    res_load(f + 1, na, nb);
                    uint32_t raw[16];
                    ptx::tmem_ld_16x256b_x4(taddr0 + ((uint32_t)(h * 16) << 16) + (uint32_t)(buf * p.BN + b * 32), raw);
                    ptx::tmem_ld_wait();
                    if (cl < p.e.cout_stride)
                        epi_quad_rows<kInt8, kPrelu>(p.e, s_scale, s_bias, cl, cq, second ? pa1 : pa0, second ? pb1 : pb0, want_res, ra,
                                                     rb, raw);
                    ra = na;
                    rb = nb;
                }
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if (kPair) ptx::mbar_arrive_cluster_u32(ptx::map_to_cta(ptx::smem_u32(&tempty_bar[buf]), 0));
                    else ptx::mbar_arrive(&tempty_bar[buf]);
                }
            }
        } else {
            const int row = q * 32 + lane;          // row of the M tile == TMEM lane
            const int tw = row % p.TW;
            const int th = (row / p.TW) % p.TH;
            const int tn = row / (p.TW * p.TH);
            const bool row_in_box = row < p.TW * p.TH * p.TN;
            const bool vec_ok = (p.e.cout_stride & 15) == 0;
            const int n_chunks = p.BN / 16;
            const bool lean = kInt8 && !kPrelu && vec_ok && p.e.out_dtype == EXB_I8 && p.e.out2_dtype < 0 &&
                              (p.e.act == EXB_ACT_NONE || p.e.act == EXB_ACT_RELU) && (p.BN & 31) == 0 && (p.e.cout_stride & 31) == 0 &&
                              (p.e.y_pitch & 31) == 0 && ((n_chunks / nsub) & 1) == 0;
            const float lean_lo = p.e.act == EXB_ACT_RELU ? 0.f : -INFINITY;
            TileCursor cur(p, first_unit + grp * unit_step, p.epi_groups * unit_step);
            for (int t = first_unit + grp * unit_step; t < total_tiles && ok; t += p.epi_groups * unit_step, ti += p.epi_groups) {
                const TileCoord tc = tile_of(cur);
                cur.advance(p);            // from here on: this group's next tile
                const int ow = tc.ow0 + tw, oh = tc.oh0 + th, n = tc.n0 + tn;
                const int buf = ti % p.acc_bufs;
                const uint32_t acc_phase = (uint32_t)(ti / p.acc_bufs) & 1u;
                const uint32_t taddr = taddr0 + (uint32_t)(buf * p.BN);
                const bool valid = row_in_box && ow < p.OW && oh < p.OH && n < p.N;
                const int64_t pix = ((int64_t)n * p.OH + oh) * p.OW + ow;
                // This warp's chunks of 16 channels.  The residual of a chunk is requested one chunk
                // ahead (the first one before the accumulator is even ready), because with so few
                // epilogue warps an exposed global-memory latency per chunk is what the epilogue costs.
                const int per = (n_chunks + nsub - 1) / nsub;
                const int c_begin = sub * per, c_end = min(n_chunks, (sub + 1) * per);
                const bool do_res = p.has_res && vec_ok && valid;
                const __half* res_row = p.e.residual + pix * p.e.cout_stride + tc.ntile * p.BN;
                uint32_t rn[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                if (!lean && do_res && c_begin < c_end && tc.ntile * p.BN + c_begin * 16 < p.e.cout_stride)
                    ld_global_nc_256(res_row + c_begin * 16, rn);
                // The residual rows of this group's NEXT tile are asked into L2 now (no register cost):
                // the tile after this one then finds them a few hundred cycles away instead of a DRAM
                // round trip per chunk, which the one-chunk-ahead register prefetch cannot cover.
                if (p.has_res && vec_ok && t + p.epi_groups * unit_step < total_tiles) {
                    const TileCoord c2 = tile_of(cur);
                    const int ow2 = c2.ow0 + tw, oh2 = c2.oh0 + th, n2 = c2.n0 + tn;
                    if (row_in_box && ow2 < p.OW && oh2 < p.OH && n2 < p.N) {
                        const __half* r2 = p.e.residual + (((int64_t)n2 * p.OH + oh2) * p.OW + ow2) * p.e.cout_stride +
                                           c2.ntile * p.BN + c_begin * 16;
                        for (int b = 0; b < (c_end - c_begin) * 32; b += 128)
                            asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(r2) + b));
                    }
                }
                if (!ptx::mbar_wait_bounded_warp(&tfull_bar[buf], acc_phase, &abort_flag, kMaxSpins)) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                if (lean) {
                    // int8-only output (with or without an fp16 residual), ReLU or no activation: 32 channels per TMEM load,
                    // the residual as two 32-byte loads and the result as one 32-byte store (whole sectors) per pixel and
                    // load, no run-time dispatch inside the loop
                    for (int chunk = c_begin; chunk < c_end; chunk += 2) {
                        const int cl = tc.ntile * p.BN + chunk * 16;
                        uint32_t r0[8] = {0, 0, 0, 0, 0, 0, 0, 0}, r1[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                        if (do_res && cl < p.e.cout_stride) {       // 32 channels of fp16 residual: two whole sectors
                            ld_global_nc_256(res_row + chunk * 16, r0);
                            ld_global_nc_256(res_row + chunk * 16 + 16, r1);
                        }
                        uint32_t raw[32];
                        ptx::tmem_ld_32x32b_x32(taddr + chunk * 16, raw);
                        ptx::tmem_ld_wait();
                        if (!valid || cl >= p.e.cout_stride) continue;
                        uint32_t o[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float4 s4 = reinterpret_cast<const float4*>(s_scale + cl)[i];
                            const float4 b4 = reinterpret_cast<const float4*>(s_bias + cl)[i];
                            const uint32_t* rr = i < 4 ? r0 : r1;
                            const float2 ra = __half22float2(*reinterpret_cast<const __half2*>(&rr[2 * (i & 3)]));
                            const float2 rb = __half22float2(*reinterpret_cast<const __half2*>(&rr[2 * (i & 3) + 1]));
                            o[i] = quant_pack4(fmaxf(epi_value<kInt8>(raw[4 * i + 0], s4.x, b4.x) + ra.x, lean_lo),
                                               fmaxf(epi_value<kInt8>(raw[4 * i + 1], s4.y, b4.y) + ra.y, lean_lo),
                                               fmaxf(epi_value<kInt8>(raw[4 * i + 2], s4.z, b4.z) + rb.x, lean_lo),
                                               fmaxf(epi_value<kInt8>(raw[4 * i + 3], s4.w, b4.w) + rb.y, lean_lo), p.e.out_scale);
                        }
                        st_global_256(static_cast<int8_t*>(p.e.y) + pix * p.e.y_pitch + cl, o);
                    }
                } else
                for (int chunk = c_begin; chunk < c_end; ++chunk) {
                    uint32_t raw[16];
                    ptx::tmem_ld_32x32b_x16(taddr + chunk * 16, raw);
                    uint32_t rc[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) rc[i] = rn[i];
                    if (do_res && chunk + 1 < c_end && tc.ntile * p.BN + (chunk + 1) * 16 < p.e.cout_stride)
                        ld_global_nc_256(res_row + (chunk + 1) * 16, rn);
                    ptx::tmem_ld_wait();
                    const int cl = tc.ntile * p.BN + chunk * 16;   // first channel of the chunk
                    if (!valid || cl >= p.e.cout_stride) continue;
                    if (vec_ok) {
                        float4 sc[4], bi[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            sc[i] = reinterpret_cast<const float4*>(s_scale + cl)[i];
                            bi[i] = reinterpret_cast<const float4*>(s_bias + cl)[i];
                        }
                        epi_row16<kInt8, kPrelu, 16, 2, 0>(p.e, sc, bi, cl, pix, do_res, rc, raw);
                    } else {
                        // ragged channel count: element-wise stores, statically indexed so the
                        // accumulators stay in registers
                        const int64_t off = pix * p.e.y_pitch + cl;
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            if (cl + i < p.e.cout_stride) {
                                float u = epi_value<kInt8>(raw[i], s_scale[cl + i], s_bias[cl + i]);
                                if (p.has_res) u += __half2float(p.e.residual[off + i]);
                                if constexpr (kPrelu) u = u >= 0.f ? u : u * __ldg(p.e.slope + cl + i);
                                else u = apply_act(u, p.e.act);
                                epi_store_scalar(p.e.y, p.e.out_dtype, off + i, u, p.e.out_scale, raw[i]);
                                if (p.e.out2_dtype >= 0)
                                    epi_store_scalar(p.e.y2, p.e.out2_dtype, off + i, u, p.e.out2_scale, raw[i]);
                            }
                        }
                    }
                }
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if (kPair) ptx::mbar_arrive_cluster_u32(ptx::map_to_cta(ptx::smem_u32(&tempty_bar[buf]), 0));
                    else ptx::mbar_arrive(&tempty_bar[buf]);
                }
            }
        }
        if (!ok && lane == 0) atomicExch(p.error, 3);
    }

    // ------------------------------- teardown -----------------------------------------------
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (kPair) ptx::cluster_sync();      // neither CTA leaves while its peer may still signal its barriers or read its TMEM
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        if (kPair) ptx::tmem_dealloc_pair(tmem_base, (uint32_t)p.tmem_cols);
        else ptx::tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
    }
}

// ---- host side ----------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    }
    return fn;
}

CUtensorMapSwizzle swizzle_for(int kb_bytes) {
    return kb_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                           : (kb_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

int round_up(int a, int b) { return (a + b - 1) / b * b; }

// Pick the pixel box (TW x TH x TN <= 128 rows) that wastes the fewest MMA rows; ties go to
// the widest box (longest contiguous runs for the TMA unit), then the tallest.
void choose_tile(int N, int OH, int OW, int& TW, int& TH, int& TN) {
    double best = -1.0;
    TW = 1; TH = 1; TN = 1;
    for (int tw = 1; tw <= OW && tw <= kTileM; ++tw)
        for (int th = 1; th <= OH && tw * th <= kTileM; ++th) {
            int tn = kTileM / (tw * th);
            if (tn > N) tn = N;
            if (tn < 1) continue;
            const int64_t tiles = (int64_t)((OW + tw - 1) / tw) * ((OH + th - 1) / th) * ((N + tn - 1) / tn);
            const double eff = (double)OW * OH * N / ((double)tiles * kTileM);
            const bool better = eff > best + 1e-9 ||
                                (eff > best - 1e-9 && (tw > TW || (tw == TW && th > TH)));
            if (better) {
                best = eff;
                TW = tw; TH = th; TN = tn;
            }
        }
}

}  // namespace

bool conv_tc_pool_fusable(const ConvGeom& g) {
    const FoldPlan fold = conv_fold_plan(g);
    const int cout_pad = (g.cout_stride + 15) / 16 * 16;
    return fold.on && g.in_dtype == EXB_F16 && g.cin_stride * 2 == 8 && g.sw == 2 && g.sh == 2 && fold.F == 8 && g.kh <= 16 &&
           cout_pad == 64 && g.cout_stride == 64 && g.out_dtype == EXB_F16 && (g.out2_dtype == -1 || g.out2_dtype == EXB_I8) &&
           !g.has_res && (g.act == EXB_ACT_RELU || g.act == EXB_ACT_RELU6) && g.group == 1;
}

bool conv_tc_eligible(const ConvGeom& g) {
    const int es = g.in_dtype == EXB_I8 ? 1 : 2;
    if (g.group != 1) return false;
    if (g.sh != g.sw || (g.sh != 1 && g.sh != 2)) return false;
    if ((g.cin_stride * es) % 32 != 0 && !conv_fold_plan(g).on) return false;   // K block of at least 32 bytes
    if (g.N < 1 || g.OH < 1 || g.OW < 1) return false;
    if (g.out_dtype == EXB_I32 && g.in_dtype != EXB_I8) return false;
    return true;
}

int conv_tc_launch(exb_ctx* ctx, const ConvGeom& g, const void* x, const exb_conv_weights* w,
                   const void* residual, void* y, void* y2, cudaStream_t st) {
    auto encode = get_encode_fn();
    if (!encode) return fail(EXB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const bool int8 = g.in_dtype == EXB_I8;
    const int es = int8 ? 1 : 2;
    ConvTcParams p;
    memset(&p, 0, sizeof(p));
    p.N = g.N; p.OH = g.OH; p.OW = g.OW;
    choose_tile(g.N, g.OH, g.OW, p.TW, p.TH, p.TN);
    p.tiles_w = (g.OW + p.TW - 1) / p.TW;
    p.tiles_h = (g.OH + p.TH - 1) / p.TH;
    p.tiles_nb = (g.N + p.TN - 1) / p.TN;
    p.step_w = p.TW; p.step_h = p.TH; p.org = 0;
    p.n_tiles = (w->cout_pad + 255) / 256;
    p.BN = round_up((w->cout_pad + p.n_tiles - 1) / p.n_tiles, 16);
    // Two CTAs per SM when the N tile is narrow (see the kernel's comment).
    bool two = p.BN <= 128;
    p.kh = g.kh; p.kw = g.kw; p.stride = g.sh; p.pad_t = g.pt; p.pad_l = g.pl;
    p.cin_pad = g.cin_stride;
    const int row_bytes = g.cin_stride * es;
    const FoldPlan fold = conv_fold_plan(g);
    p.fold = fold.on ? 1 : 0;
    if (fold.on) {
        p.kb_bytes = fold.kb_bytes;
        p.kb_elems = p.kb_bytes / es;
        p.cblks = 1;
    } else {
        p.kb_bytes = row_bytes % 128 == 0 ? 128 : (row_bytes % 64 == 0 ? 64 : 32);
        p.kb_elems = p.kb_bytes / es;
        p.cblks = row_bytes / p.kb_bytes;
    }
    p.a_bytes = kTileM * p.kb_bytes;
    p.b_bytes = p.BN * p.kb_bytes;
    // Patch mode (see ConvTcParams): stride-2 fp16 stems on 8-byte pixels with an 8-pixel window.
    const bool patch = fold.on && !int8 && g.cin_stride * es == 8 && g.sw == 2 && fold.F == 8 && p.n_tiles == 1 &&
                       g.kh <= 16;
    p.patch = patch ? 1 : 0;
    if (patch) {
        p.TW = 8; p.TH = 16; p.TN = 1;   // 16 groups of 8 output columns, one output row each
        p.tiles_w = (g.OW + 7) / 8;
        p.tiles_h = (g.OH + 15) / 16;
        p.tiles_nb = g.N;
        p.patch_rows = 2 * p.TH + g.kh - 2;
        p.patch_pitch = (2 * p.TW + 8) * 8;   // 2*TW + 6 pixels needed, rounded to 24
        p.a_bytes = round_up(p.patch_rows * p.patch_pitch, 128);
        p.w_global = w->d_w;
        p.step_w = p.TW; p.step_h = p.TH;
        if (g.pool) {
            p.pool = 1;
            p.PH = g.PH; p.PW = g.PW;
            p.step_w = p.TW - 2; p.step_h = p.TH - 2; p.org = -1;
            p.tiles_w = (g.PW + 2) / 3;      // 3 x 7 pooled outputs per tile
            p.tiles_h = (g.PH + 6) / 7;
        }
    }
    if (g.pool && !(patch && two && p.BN == 64 && conv_tc_pool_fusable(g)))
        return fail(EXB_ERR_UNSUPPORTED, "fused pooling needs the patch-mode stem kernel with 64 output channels");
    p.a_tx_bytes = p.TW * p.TH * p.TN * p.kb_bytes;
    p.taps = 1;
    p.a_sbo = 8 * p.kb_bytes;
    // Row-box mode (see ConvTcParams): stride 1, at least two taps per kernel row, dense input rows.  The tile is 8
    // pixels wide; TH x TN = 16 is chosen for the fewest wasted rows.  Taken when it moves fewer operand bytes from L2
    // into shared memory than the tap-by-tap loop does, counting the extra tiles a map whose width is not a multiple
    // of 8 costs and the weights that stay resident.
    struct RowBox {
        bool on;
        int TH, TN, one_cta;
    } rb = {false, 0, 0, 0};
    if (!fold.on && !patch && g.sh == 1 && g.sw == 1 && g.kw >= 2 && g.kw <= 9 && g.w_pitch == g.W && g.w_pad == 0 &&
        p.kb_bytes >= 64) {      // 32-byte K rows: measured slower than the tap loop (0.190 vs 0.162 ms, 16 -> 32 channels @320)
        double best = -1.0;
        for (int th = 16; th >= 1; th >>= 1) {
            const int tn = 16 / th;
            const int64_t tiles = (int64_t)((g.OH + th - 1) / th) * ((g.N + tn - 1) / tn);
            const double eff = (double)g.OH * g.N / ((double)tiles * th * tn);
            if (eff > best + 1e-9) {
                best = eff;
                rb.TH = th;
                rb.TN = tn;
            }
        }
        const int64_t tiles_rb = (int64_t)((g.OW + 7) / 8) * ((g.OH + rb.TH - 1) / rb.TH) * ((g.N + rb.TN - 1) / rb.TN);
        const int64_t tiles_tap = (int64_t)p.tiles_w * p.tiles_h * p.tiles_nb;
        const int64_t k_bytes_all = (int64_t)g.kh * g.kw * p.cblks * p.kb_bytes;             // K bytes of one operand row
        const int64_t a_tap = kTileM * k_bytes_all;
        const int64_t a_rb = (int64_t)(8 + g.kw - 1) * 16 * g.kh * p.cblks * p.kb_bytes;
        const int64_t b_tile = (int64_t)p.BN * k_bytes_all;
        // weights stay resident with two CTAs per SM (as before) or, in row-box mode, with one CTA per SM as well
        const bool res_two = p.n_tiles == 1 && two && b_tile <= 48 * 1024;
        const bool res_one = p.n_tiles == 1 && b_tile <= 150 * 1024;
        // One CTA per SM (to keep the weights resident) only for N tiles of 128 and more: a single issuing thread
        // cannot keep the tensor pipe busy with N = 64 instructions.
        const bool one_cta = res_one && !res_two && two && p.BN >= 128;
        const bool res_rb = (two && !one_cta) ? res_two : res_one;
        const double cost_tap = (double)tiles_tap * (a_tap + (res_two ? 0 : b_tile));
        const double cost_rb = (double)tiles_rb * (a_rb + (res_rb ? 0 : b_tile));
        if (cost_rb < 0.85 * cost_tap) {
            rb.on = true;
            rb.one_cta = one_cta ? 1 : 0;
            // at least three units must fit beside the tables (and the resident weights)
            const bool two_rb = two && !rb.one_cta;
            const int64_t room = (two_rb ? 228 * 1024 / 2 - 1024 : ctx->smem_optin) - 2048 - 2 * p.n_tiles * p.BN * (int)sizeof(float) -
                                 g.kh * p.cblks * (int)sizeof(int4);
            const bool res = two_rb ? res_two : res_one;
            const int64_t unit = round_up((8 + g.kw - 1) * 16 * p.kb_bytes, 1024) + (res ? 0 : (int64_t)g.kw * p.b_bytes);
            if (room - (res ? b_tile : 0) < 3 * unit) rb.on = false;
        }
    }
    if (rb.on) {
        p.rowbox = 1;
        p.taps = g.kw;
        p.TW = 8; p.TH = rb.TH; p.TN = rb.TN;
        p.tiles_w = (g.OW + 7) / 8;
        p.tiles_h = (g.OH + p.TH - 1) / p.TH;
        p.tiles_nb = (g.N + p.TN - 1) / p.TN;
        p.step_w = p.TW; p.step_h = p.TH; p.org = 0;
        p.a_sbo = (8 + g.kw - 1) * p.kb_bytes;
        p.a_bytes = (8 + g.kw - 1) * 16 * p.kb_bytes;      // one box: a multiple of 1024 bytes for every kb_bytes >= 64
        p.a_bytes = round_up(p.a_bytes, 1024);
        p.a_tx_bytes = (8 + g.kw - 1) * 16 * p.kb_bytes;
        if (rb.one_cta) two = false;
    }
    const int ctas_per_sm = two ? 2 : 1;
    // CTA pairs (see the kernel's kPair): N tiles of 256 on one CTA per SM in the plain tap loop, and N tiles of 128
    // in the row-box loop with resident weights (each CTA then keeps half of them and a stage can hold a whole tile);
    // at least two image groups to pair up.  Each CTA holds half of the tile's weight rows.
    const bool pair = !two && !patch && !fold.on && !g.pool && p.tiles_nb >= 2 && ctx->sm_count >= 2 && g.act != EXB_ACT_PRELU &&
                      (p.rowbox ? (p.BN == 128 && p.n_tiles == 1 && rb.one_cta) : p.BN == 256);
    if (pair) p.b_bytes = (p.BN / 2) * p.kb_bytes;
    const int k_iters = fold.on ? g.kh : (p.rowbox ? g.kh * p.cblks : g.kh * g.kw * p.cblks);
    p.k_iters = k_iters;
    if ((int64_t)g.N * g.OH * g.OW >= (int64_t)1 << 31) return fail(EXB_ERR_UNSUPPORTED, "more than 2^31 output pixels");
    if ((int64_t)g.kh * w->kw_pack * w->cin_pad >= (1 << 28)) return fail(EXB_ERR_UNSUPPORTED, "reduction dimension too large");
    const int epi_bytes = 2 * p.n_tiles * p.BN * (int)sizeof(float) + k_iters * (int)sizeof(int4) +
                          (g.pool ? 2 * kTileM * 128 : 0);
    // static barriers + alignment slack + tables; two resident CTAs share the SM's 228 KB
    // (1 KB of which is reserved per CTA)
    int budget = (two ? (228 * 1024 / 2 - 1024) : ctx->smem_optin) - 2048 - epi_bytes;
    // Keep the weights in shared memory for the whole kernel when the slice fits beside a useful
    // operand ring: it removes the weight re-read per tile from the L2 -> SM traffic that bounds
    // this kernel.
    const int b_all = k_iters * p.taps * p.b_bytes;
    p.b_resident = ((!pair || p.rowbox) && p.n_tiles == 1 && b_all <= 150 * 1024 && budget - b_all >= (p.rowbox ? 3 : 4) * p.a_bytes) ? 1 : 0;
    if (p.b_resident) budget -= b_all;
    const int blk_bytes = p.a_bytes + (p.b_resident ? 0 : p.taps * p.b_bytes);
    // K blocks per stage: aim at ~48 KB stages (one mbarrier round trip each), keep >= 3 stages,
    // prefer a group size that divides the K loop.
    int gmax = (48 * 1024) / blk_bytes;
    if (gmax < 1) gmax = 1;
    if (gmax > 16) gmax = 16;
    if (gmax > k_iters) gmax = k_iters;
    int G = gmax;
    for (int gcand = gmax; gcand >= (gmax + 1) / 2 && gcand >= 1; --gcand)
        if (k_iters % gcand == 0) {
            G = gcand;
            break;
        }
    while (G > 1 && budget / (G * blk_bytes) < 3) --G;
    if (pair) {
        // One thread issues for two SMs: every commit and barrier wait it spends idles both tensor pipes, so a stage
        // carries as many K blocks as two stages allow (three 32 KB blocks of A + half-B).  Measured on the 256 / 512-
        // channel layers: pairs with one block per stage 0.038 ms, with three 0.031 ms, single CTAs 0.035 ms.
        G = 1;
        for (int cand = 2; cand <= 4; ++cand)
            if (k_iters % cand == 0 && budget / (cand * blk_bytes) >= 2) G = cand;
    }
    if (p.rowbox) {
        // A row-box unit already carries kw taps.  One stage per tile (all its units behind one barrier and one
        // commit) when two such stages fit - every hand-over costs the single issuing thread a few hundred
        // cycles - else one unit per stage and as many stages as fit.
        G = (k_iters * blk_bytes <= (pair ? 96 : 48) * 1024 && budget / (k_iters * blk_bytes) >= 2) ? k_iters : 1;
    }
    p.kgroup = G;
    int stages = budget / (G * blk_bytes);
    if (patch) {   // ring of whole patches, weights in their own region
        p.kgroup = G = 1;
        if (p.b_resident) budget += b_all;
        p.b_resident = 0;
        stages = (budget - g.kh * p.BN * 64) / p.a_bytes;
    }
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < 2) return fail(EXB_ERR_UNSUPPORTED, "conv tile does not fit shared memory (BN=%d)", p.BN);
    p.b_region = patch ? g.kh * p.BN * 64 : (p.b_resident ? b_all : stages * G * p.taps * p.b_bytes);
    p.stages = stages;
    // As many accumulator buffers as TMEM allows (256 columns per CTA with two CTAs per SM, else
    // 512): a buffer goes round MMA -> hand-over -> epilogue -> hand-back, and the two hand-overs
    // alone cost a couple of microseconds, so the number of buffers in flight sets the tile rate
    // of short layers.  Epilogue groups need four warps each (one per TMEM lane quarter).
    p.acc_bufs = two ? (p.BN <= 64 ? 4 : 2) : (p.BN <= 128 ? 4 : 2);
    if (patch && g.pool) {     // patch ring and accumulator ring run in lockstep (see the producer)
        if (p.stages < p.acc_bufs) return fail(EXB_ERR_UNSUPPORTED, "patch ring does not fit shared memory (BN=%d)", p.BN);
        p.stages = p.acc_bufs;
    }
    p.epi_groups = two ? 2 : (p.acc_bufs == 4 ? 4 : 2);
    int cols = 32;
    while (cols < p.acc_bufs * p.BN) cols *= 2;
    p.tmem_cols = cols;
    p.idesc = ptx::make_idesc(int8, pair ? 2 * kTileM : kTileM, (uint32_t)p.BN);
    p.cout_pad = w->cout_pad;
    p.has_res = g.has_res;
    p.e.scale = w->d_scale; p.e.bias = w->d_bias; p.e.slope = w->d_slope; p.e.residual = static_cast<const __half*>(residual);
    p.e.y = y; p.e.y2 = y2; p.e.out_dtype = g.out_dtype; p.e.out2_dtype = g.out2_dtype; p.e.act = g.act;
    p.e.out_scale = g.out_scale; p.e.out2_scale = g.out2_scale; p.e.cout_stride = g.cout_stride; p.e.y_pitch = g.y_pitch;
    p.error = ctx->d_error;
    if (g.pool) {       // BN == 64 (checked above)
        for (int c = 0; c < kConstCh; ++c) {
            p.c_scale[c] = c < w->cout_pad ? w->h_scale[c] : 0.f;
            p.c_bias[c] = c < w->cout_pad ? w->h_bias[c] : 0.f;
        }
    }

    const CUtensorMapDataType dt = int8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUtensorMapSwizzle sw = swizzle_for(p.kb_bytes);
    // A: one view per input parity (only view 0 for stride 1).  Rows may be physically padded.
    const size_t px_bytes = (size_t)g.cin_stride * es;
    const size_t row_pitch = (size_t)g.w_pitch * px_bytes;
    const int nviews = g.sh == 1 ? 1 : 4;
    if (patch) {
        // One map: whole padded rows as the innermost dimension, box = 24 pixels x patch_rows.
        cuuint64_t dims[3] = {(cuuint64_t)g.w_pitch * g.cin_stride, (cuuint64_t)g.H, (cuuint64_t)g.N};
        cuuint64_t strides[2] = {(cuuint64_t)row_pitch, (cuuint64_t)g.H * row_pitch};
        cuuint32_t box[3] = {(cuuint32_t)(p.patch_pitch / es), (cuuint32_t)p.patch_rows, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        void* base = const_cast<char*>(static_cast<const char*>(x)) + (size_t)(g.w_pad - fold.pl_eff) * px_bytes;
        CUresult r = encode(&p.tmA[0], dt, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(EXB_ERR_CUDA, "cuTensorMapEncodeTiled(patch) failed with %d", (int)r);
    }
    for (int v = 0; v < (patch ? 0 : nviews); ++v) {
        const int ph = v >> 1, pw = v & 1;
        const int st_ = g.sh;
        if (fold.on && pw) continue;   // the folded layout walks W inside the K row
        // rows / columns of this view: indices ph, ph+st, ... < H
        const int vh = (g.H - ph + st_ - 1) / st_;
        const int vw = (g.W - pw + st_ - 1) / st_;
        if (vh <= 0 || vw <= 0) return fail(EXB_ERR_UNSUPPORTED, "stride-2 convolution needs H and W of at least 2");
        CUresult r;
        if (fold.on) {
            // dim0: F pixels x cin_stride channels (one K row), dim1: output columns, stepping
            // stride_w pixels (windows of neighbouring columns overlap), dim2: rows of this parity.
            cuuint64_t dims[4] = {(cuuint64_t)p.kb_elems, (cuuint64_t)g.OW, (cuuint64_t)vh, (cuuint64_t)g.N};
            cuuint64_t strides[3] = {(cuuint64_t)g.sw * px_bytes, (cuuint64_t)st_ * row_pitch, (cuuint64_t)g.H * row_pitch};
            cuuint32_t box[4] = {(cuuint32_t)p.kb_elems, (cuuint32_t)p.TW, (cuuint32_t)p.TH, (cuuint32_t)p.TN};
            cuuint32_t estr[4] = {1, 1, 1, 1};
            void* base = const_cast<char*>(static_cast<const char*>(x)) + (size_t)ph * row_pitch +
                         (size_t)(g.w_pad - fold.pl_eff) * px_bytes;
            r = encode(&p.tmA[v], dt, 4, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        } else {
            cuuint64_t dims[4] = {(cuuint64_t)g.cin_stride, (cuuint64_t)vw, (cuuint64_t)vh, (cuuint64_t)g.N};
            cuuint64_t strides[3] = {(cuuint64_t)st_ * px_bytes, (cuuint64_t)st_ * row_pitch, (cuuint64_t)g.H * row_pitch};
            cuuint32_t box[4] = {(cuuint32_t)p.kb_elems, (cuuint32_t)(p.rowbox ? p.TW + g.kw - 1 : p.TW), (cuuint32_t)p.TH,
                                 (cuuint32_t)p.TN};
            cuuint32_t estr[4] = {1, 1, 1, 1};
            void* base = const_cast<char*>(static_cast<const char*>(x)) + (size_t)ph * row_pitch +
                         (size_t)(pw + g.w_pad) * px_bytes;
            r = encode(&p.tmA[v], dt, 4, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        }
        if (r != CUDA_SUCCESS) return fail(EXB_ERR_CUDA, "cuTensorMapEncodeTiled(A view %d) failed with %d", v, (int)r);
    }
    // Quad epilogue: N tiles of whole 32-channel blocks, every channel group of 8 either fully inside the output or
    // fully outside, weights stored in whole 32-row blocks (the permuting map walks rows 32 at a time).  Taken when
    // the epilogue moves fp16 / fp32 data (an fp16 output or residual): there its whole-sector accesses are worth
    // 15-20 % of the layer; a lone int8 output is as fast from the thread-per-pixel epilogue (measured on the
    // ResNet-18-style layers at batch 256), which needs fewer TMEM loads.
    const bool quad = !patch && !p.pool && p.BN % 32 == 0 && w->cout_pad % 32 == 0 && (g.cout_stride & 7) == 0 &&
                      g.out_dtype != EXB_I32 && !(g.out_dtype == EXB_I8 && g.out2_dtype < 0) &&
                      p.TW <= 255 && p.TH <= 255 && p.TN <= 32767;
    p.b_perm = quad ? 1 : 0;
    {
        const int K = g.kh * w->kw_pack * w->cin_pad;
        CUresult r;
        if (quad) {
            // Rows of the packed matrix [cout][K] seen as (e: 2, j: 4, g: 4, block) with row = 32*block + 8*j + 2*g + e,
            // traversed e, j, g, block: shared-memory row (= accumulator column) 8*g + 2*j + e of a block holds
            // output channel 8*j + 2*g + e.
            const cuuint64_t kb = (cuuint64_t)K * es;
            cuuint64_t dims[5] = {(cuuint64_t)K, 2, 4, 4, (cuuint64_t)(w->cout_pad / 32)};
            cuuint64_t strides[4] = {kb, 8 * kb, 2 * kb, 32 * kb};
            cuuint32_t box[5] = {(cuuint32_t)p.kb_elems, 2, 4, 4, (cuuint32_t)((pair ? p.BN / 2 : p.BN) / 32)};
            cuuint32_t estr[5] = {1, 1, 1, 1, 1};
            r = encode(&p.tmB, dt, 5, w->d_w, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        } else {
            cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)w->cout_pad};
            cuuint64_t strides[1] = {(cuuint64_t)K * es};
            cuuint32_t box[2] = {(cuuint32_t)p.kb_elems, (cuuint32_t)(pair ? p.BN / 2 : p.BN)};
            cuuint32_t estr[2] = {1, 1};
            r = encode(&p.tmB, dt, 2, w->d_w, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        }
        if (r != CUDA_SUCCESS) return fail(EXB_ERR_CUDA, "cuTensorMapEncodeTiled(B) failed with %d", (int)r);
    }

    const int total_tiles = p.tiles_w * p.tiles_h * p.tiles_nb * p.n_tiles;
    const int max_ctas = ctx->sm_count * ctas_per_sm;
    int grid = total_tiles < max_ctas ? total_tiles : max_ctas;
    if (pair) {      // clusters of two CTAs, one per pair of tiles
        const int pairs = p.tiles_w * p.tiles_h * ((p.tiles_nb + 1) / 2) * p.n_tiles;
        const int clusters = pairs < ctx->sm_count / 2 ? pairs : ctx->sm_count / 2;
        grid = 2 * clusters;
    }
    const size_t smem = (size_t)p.stages * p.kgroup * p.a_bytes + p.b_region + 1024 + epi_bytes;
    const bool prelu = p.e.act == EXB_ACT_PRELU;
    void (*kern)(const ConvTcParams);
    if (p.pool) kern = conv_tc_kernel<false, 8, kEpiPool>;
    else if (pair && !prelu)
        kern = int8 ? (quad ? conv_tc_kernel<true, 16, kEpiQuad, false, true> : conv_tc_kernel<true, 16, kEpiRow, false, true>)
                    : (quad ? conv_tc_kernel<false, 16, kEpiQuad, false, true> : conv_tc_kernel<false, 16, kEpiRow, false, true>);
    else if (quad && !prelu)
        kern = int8 ? (two ? conv_tc_kernel<true, 8, kEpiQuad> : conv_tc_kernel<true, 16, kEpiQuad>)
                    : (two ? conv_tc_kernel<false, 8, kEpiQuad> : conv_tc_kernel<false, 16, kEpiQuad>);
    else if (quad)
        kern = int8 ? (two ? conv_tc_kernel<true, 8, kEpiQuad, true> : conv_tc_kernel<true, 16, kEpiQuad, true>)
                    : (two ? conv_tc_kernel<false, 8, kEpiQuad, true> : conv_tc_kernel<false, 16, kEpiQuad, true>);
    else if (!prelu)
        kern = int8 ? (two ? conv_tc_kernel<true, 8, kEpiRow> : conv_tc_kernel<true, 16, kEpiRow>)
                    : (two ? conv_tc_kernel<false, 8, kEpiRow> : conv_tc_kernel<false, 16, kEpiRow>);
    else
        kern = int8 ? (two ? conv_tc_kernel<true, 8, kEpiRow, true> : conv_tc_kernel<true, 16, kEpiRow, true>)
                    : (two ? conv_tc_kernel<false, 8, kEpiRow, true> : conv_tc_kernel<false, 16, kEpiRow, true>);
    // The dynamic shared-memory limit is an attribute of the kernel function on a device, shared by every thread that
    // launches it: it is raised to the device's maximum once, never lowered, so that concurrent launches from several
    // host threads (one pipeline replica per thread) cannot undercut each other.  Occupancy follows the bytes a launch
    // actually asks for, not this limit.
    {
        static std::mutex attr_mutex;
        static std::set<std::pair<const void*, int>> raised;
        std::lock_guard<std::mutex> lock(attr_mutex);
        const auto key = std::make_pair(reinterpret_cast<const void*>(kern), ctx->device);
        if (!raised.count(key)) {
            cudaFuncAttributes fa;
            EXB_CUDA_TRY(cudaFuncGetAttributes(&fa, kern));      // static + dynamic shared memory share the device limit
            EXB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              ctx->smem_optin - (int)fa.sharedSizeBytes));
            raised.insert(key);
        }
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)((kFirstEpiWarp + (two ? 8 : 16)) * 32));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (ctx->pdl) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (pair) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = 2;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    EXB_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
    return after_launch("conv_tc_kernel");
}

}  // namespace exb
