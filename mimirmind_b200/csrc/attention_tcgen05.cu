// Paged causal prefill attention on the tcgen05 tensor cores, head sizes 64 and 128, bfloat16.
//
// One CTA per (tile of up to 128 query tokens of one request, query head).  Q stays in shared
// memory; keys and values stream in tiles of 128 keys, fetched page by page with TMA straight
// from the page pool (in this cache layout one page of one KV head is one contiguous
// [page_size, head size] block).  Per key tile (head size 128; with 64 the products have half the depth or width):
//     S  = Q K^T          tcgen05.mma 128x128x16 x 8, both operands K-major, S in tensor memory
//     softmax             two groups of 128 threads, one thread per query row in each: group 0 takes the even
//                         key tiles, group 1 the odd ones, each with a maximum, a sum and an O accumulator of
//                         its own (merged at the end), so no thread ever waits for another thread's maximum
//                         and one group's exponentials overlap the other group's loads, masks and stores:
//                         tcgen05.ld of the row, mask by position, P rounded to bf16 into shared memory in
//                         the 128-byte-swizzled K-major layout the tensor core reads
//     O[g] += P V         tcgen05.mma 128x128x16 x 8, V read MN-major (as stored: keys x head dim), accumulated
//                         in tensor memory over all key tiles of the group
// O is rescaled lazily: probabilities are taken relative to a reference maximum that is only moved (and O, in
// tensor memory, multiplied by the matching factor with tcgen05.ld / tcgen05.st) when the row's maximum has grown
// by more than 2^8 since; until then P may exceed 1 by that factor, which bf16 and the fp32 sums hold easily.
// After the first few tiles a row's maximum rarely grows that much, so the threads neither read nor scale O per
// tile.  S and P are double-buffered: while the softmax threads work on tile t the tensor core already computes S
// of tile t+1 and adds P V of tile t-1.
// Warp 1 issues Q K^T, warp 11 issues P V (a single issuing thread, waiting on the barriers of both products in
// turn, was what bound the kernel); warp 0 = TMA producer for keys (and Q), warp 10 = TMA producer for values: every lane fetches one half of one
// page, so the 16 to 32 small copies of a tile are issued at once (one thread issuing them in turn was the
// bottleneck of the whole kernel); warp 1 = MMA issuer and tensor-memory owner; warps 2..9 = softmax and output.  Same formula as the other attention kernels (reference src/compute/Attention.cpp:43-94).
// Warp 0 requests Q and the first key tile before the CTA's set-up barrier (tensor-memory allocation, zeroing of the value
// ring), which nothing of that needs.
// All mbarrier waits are bounded; on a time-out the kernel frees its tensor memory, sets `err`
// and returns.
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int BM = 128;          // query rows per CTA (tensor-memory lanes)
constexpr int BN = 128;          // keys per tile
constexpr int KV_STAGES = 2;
constexpr int HALF_BYTES = 128 * 64 * 2;        // a [128 rows x 64 columns] bf16 sub-tile, 128 bytes per row
constexpr int TILE_BYTES = 2 * HALF_BYTES;      // [128 x 128] as two column halves: a tile of P
constexpr int ATT_TC_THREADS = 384;            // K producer warp, Q K^T issuer, 8 softmax warps, V producer warp, P V issuer
constexpr int V_PRODUCER_WARP = 10;
constexpr int PV_ISSUER_WARP = 11;             // the two products have issuers of their own: each waits on its own barriers
constexpr int SOFTMAX_WARPS = 8;               // two groups of four
constexpr int GROUP_WARPS = 4;                 // barriers between the softmax warps and the tensor core count warps, not
                                               // threads: one arrival per softmax warp on one mbarrier serialise and cost more than the math
constexpr int TMEM_COLS_ATT = 512;              // S of the even / odd tiles: columns 0..255; O of the even / odd tiles: from 256, head-size columns each
constexpr float RESCALE_STEP = 8.0f;            // log2 of how far a row's maximum may run ahead of its reference

struct AttCtl {
    uint64_t q_full;
    uint64_t k_full[KV_STAGES];     // keys and values have rings of their own: a key tile is free as soon as Q K^T has read
    uint64_t k_empty[KV_STAGES];    // it, so the next keys are fetched a whole tile earlier than if they waited for P V
    uint64_t v_full[KV_STAGES];
    uint64_t v_empty[KV_STAGES];
    uint64_t s_full[2];      // S buffer b holds Q K^T of a tile (tensor core -> softmax)
    uint64_t s_free[2];      // ... has been read (softmax -> tensor core), one arrival per softmax warp
    uint64_t p_full[2];      // P buffer b is written and fenced (softmax -> tensor core), one arrival per softmax warp
    uint64_t pv_done[2];     // P V of a tile with parity b has been added into O: P buffer b is free, O is at rest until
                             // the next P is published (tensor core -> softmax)
    uint32_t tmem_base;
    int abort_flag;
    uint64_t l_full;         // both groups have posted each row's reference maximum and sum (one arrival per softmax warp)
    float xchg[2][2][128];   // [group][maximum, sum][row]
};

__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
                   "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 2^x on the special-function unit in one instruction (relative error 2^-22, far below the bf16 rounding of P)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Every lane has done its part (and its fences); one lane arrives for the warp.
__device__ __forceinline__ void warp_arrive(uint32_t bar, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
}

// tiles: int32 [n_tiles, 4] = (request index, first token row, rows in the tile (<= 128), position of the first row)
template <int HD>
__global__ void __launch_bounds__(ATT_TC_THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                            const __grid_constant__ CUtensorMap tmV, __nv_bfloat16* __restrict__ out,
                            const int32_t* __restrict__ tiles, const int32_t* __restrict__ block_table, int table_width,
                            int page_size, int H, int G, int window, float scale_log2, int* __restrict__ err) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];   // 128-byte swizzle wants 1024-byte aligned tiles
    if ((smem_u32(smem_raw) & 1023u) != 0) {                      // never seen; without the alignment nothing below is valid
        if (threadIdx.x == 0 && err != nullptr) atomicExch(err, 3);
        return;
    }
    constexpr int HALVES = HD / 64;                             // 64-column halves of a row of Q, K or V
    constexpr int HEAD_TILE_BYTES = HALVES * HALF_BYTES;        // [128 rows x head size]: a tile of Q, of keys or of values
    unsigned char* sQ = smem_raw;                               // HEAD_TILE_BYTES
    unsigned char* sP = sQ + HEAD_TILE_BYTES;                   // 2 * TILE_BYTES
    unsigned char* sK = sP + 2 * TILE_BYTES;                    // KV_STAGES * HEAD_TILE_BYTES
    unsigned char* sV = sK + KV_STAGES * HEAD_TILE_BYTES;       // KV_STAGES * HEAD_TILE_BYTES
    AttCtl* ctl = reinterpret_cast<AttCtl*>(sV + KV_STAGES * HEAD_TILE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = &ctl->abort_flag;

    // heads fastest, later (longer) tiles first: the longest tiles of every head start in the first wave
    const int tile = gridDim.y - 1 - blockIdx.y, h = blockIdx.x;
    const int g = (h * G) / H;
    const int req = tiles[tile * 4 + 0], row0 = tiles[tile * 4 + 1], n_rows = tiles[tile * 4 + 2], pos0 = tiles[tile * 4 + 3];
    const int32_t* table = block_table + (size_t)req * table_width;
    const int hi_all = pos0 + n_rows;
    const int lo_all = (window > 0 && pos0 + 1 > window) ? pos0 + 1 - window : 0;
    const int kt_begin = lo_all / BN, kt_end = (hi_all + BN - 1) / BN;

    if (threadIdx.x == 64) {
        prefetch_tensormap(&tmQ);
        prefetch_tensormap(&tmK);
        prefetch_tensormap(&tmV);
    }
    // ---- what the TMA producers need: warp 0 keys (and Q), warp 10 values; lane = (page of the tile, column half) ----
    const int pages_per_tile = BN / page_size;
    const uint32_t page_bytes = (uint32_t)page_size * 128u;           // one column half of a page
    const int pj = lane / HALVES, phf = lane % HALVES;                // this lane's page and half
    // pages of a tile that hold keys some row of the tile may see.  The ids are read a few tiles ahead: the load
    // from the block table would otherwise sit, with its full latency, between every two tiles.
    auto page_of = [&](int kt) -> int {
        if (kt >= kt_end || pj >= pages_per_tile) return -1;
        const int key_lo = kt * BN + pj * page_size;
        return (key_lo < hi_all && key_lo + page_size > lo_all) ? table[kt * pages_per_tile + pj] : -1;
    };
    constexpr int AHEAD = 4;
    int ahead[AHEAD];
    // one tile of keys or values: waits for the stage (not for the very first round), announces the bytes, copies
    auto produce = [&](bool for_k, int kt, uint32_t it, bool wait) -> bool {
        const int s = it % KV_STAGES;
        const uint32_t ph = (it / KV_STAGES) & 1;
        const int pid = ahead[0];
#pragma unroll
        for (int i = 0; i + 1 < AHEAD; ++i) ahead[i] = ahead[i + 1];
        ahead[AHEAD - 1] = page_of(kt + AHEAD);
        const uint32_t have = __ballot_sync(0xffffffffu, pid >= 0);
        const uint32_t full = smem_u32(for_k ? &ctl->k_full[s] : &ctl->v_full[s]);
        bool ok = true;
        if (lane == 0) {
            if (wait) ok = mbar_wait(smem_u32(for_k ? &ctl->k_empty[s] : &ctl->v_empty[s]), ph ^ 1, abort_flag);
            if (ok) mbar_expect_tx(full, (uint32_t)__popc(have) * page_bytes);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok && pid >= 0)
            tma_load_2d(smem_u32((for_k ? sK : sV) + s * HEAD_TILE_BYTES) + phf * HALF_BYTES + (uint32_t)pj * page_bytes, for_k ? &tmK : &tmV,
                        phf * 64, (pid * G + g) * page_size, full);
        return ok;
    };
    if (warp == 0 || warp == V_PRODUCER_WARP) {
#pragma unroll
        for (int i = 0; i < AHEAD; ++i) ahead[i] = page_of(kt_begin + i);
    }
    if (warp == 0) {
        if (lane == 0) {
            mbar_init(smem_u32(&ctl->q_full), 1);
            for (int s = 0; s < KV_STAGES; ++s) {
                mbar_init(smem_u32(&ctl->k_full[s]), 1);
                mbar_init(smem_u32(&ctl->k_empty[s]), 1);
                mbar_init(smem_u32(&ctl->v_full[s]), 1);
                mbar_init(smem_u32(&ctl->v_empty[s]), 1);
            }
            for (int b = 0; b < 2; ++b) {
                mbar_init(smem_u32(&ctl->s_full[b]), 1);
                mbar_init(smem_u32(&ctl->s_free[b]), GROUP_WARPS);
                mbar_init(smem_u32(&ctl->p_full[b]), GROUP_WARPS);
                mbar_init(smem_u32(&ctl->pv_done[b]), 1);
            }
            mbar_init(smem_u32(&ctl->l_full), SOFTMAX_WARPS);
            ctl->abort_flag = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            // Q and the first tile of keys need nobody else: their copies go out before the CTA has set itself up
            const uint32_t qbar = smem_u32(&ctl->q_full);
            mbar_expect_tx(qbar, HEAD_TILE_BYTES);
#pragma unroll
            for (int hf = 0; hf < HALVES; ++hf) tma_load_2d(smem_u32(sQ) + hf * HALF_BYTES, &tmQ, h * HD + hf * 64, row0, qbar);
        }
        __syncwarp();
        if (kt_begin < kt_end) produce(true, kt_begin, 0, false);
    }
    // Value tiles must never hold non-finite leftovers: rows of a page that was not fetched are multiplied by P = 0.
    for (int i = threadIdx.x; i < KV_STAGES * HEAD_TILE_BYTES / 16; i += ATT_TC_THREADS) reinterpret_cast<uint4*>(sV)[i] = make_uint4(0, 0, 0, 0);
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(TMEM_COLS_ATT) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;

    if (warp == 0 || warp == V_PRODUCER_WARP) {
        // ---- TMA producers ----
        const bool for_k = warp == 0;
        bool ok = true;
        uint32_t it = for_k ? 1u : 0u;                                 // the first key tile is on its way already
        for (int kt = kt_begin + (int)it; kt < kt_end && ok; ++kt, ++it) ok = produce(for_k, kt, it, true);
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer ----
            constexpr uint32_t IDESC_QK = idesc_bf16(BM, BN, false);
            const int n_tiles_k = kt_end - kt_begin;
            const uint32_t q_addr = smem_u32(sQ);
            bool ok = mbar_wait(smem_u32(&ctl->q_full), 0, abort_flag);
            // S[it % 2] = Q K(it)^T; the buffer was last read by the softmax of tile it - 2
            auto issue_qk = [&](uint32_t it) -> bool {
                const int s = it % KV_STAGES;
                const uint32_t b = it & 1, u = it >> 1;
                if (!mbar_wait(smem_u32(&ctl->s_free[b]), (u & 1) ^ 1, abort_flag)) return false;
                if (!mbar_wait(smem_u32(&ctl->k_full[s]), (it / KV_STAGES) & 1, abort_flag)) return false;
                tc_fence_after();
                const uint32_t k_addr = smem_u32(sK + s * HEAD_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * HALF_BYTES + (k & 3) * 32;      // 16 columns = 32 bytes inside the swizzled row
                    umma_bf16(tmem_base + b * 128, smem_desc_sw128(q_addr + off, 16, 1024), smem_desc_sw128(k_addr + off, 16, 1024), IDESC_QK, k ? 1u : 0u);
                }
                umma_commit(smem_u32(&ctl->s_full[b]));
                umma_commit(smem_u32(&ctl->k_empty[s]));        // the key tile is free once these products have read it
                return true;
            };
            // Two tiles ahead: S of tile it + 2 goes where S of tile it was as soon as its group has taken that into
            // registers (early in its work on tile it), so S of a group's next tile is there when it comes for it.
            for (uint32_t it = 0; (int)it < n_tiles_k && ok; ++it) ok = issue_qk(it);
        }
    } else if (warp == PV_ISSUER_WARP) {
        if (lane == 0) {
            // ---- P V issuer ----
            constexpr uint32_t IDESC_PV = idesc_bf16(BM, HD, true);
            const int n_tiles_k = kt_end - kt_begin;
            for (uint32_t it = 0; (int)it < n_tiles_k; ++it) {
                const int s = it % KV_STAGES;
                const uint32_t b = it & 1, u = it >> 1;
                if (!mbar_wait(smem_u32(&ctl->p_full[b]), u & 1, abort_flag)) break;       // P is there, O is rescaled
                if (!mbar_wait(smem_u32(&ctl->v_full[s]), (it / KV_STAGES) & 1, abort_flag)) break;
                tc_fence_after();
                const uint32_t p_addr = smem_u32(sP + b * TILE_BYTES), v_addr = smem_u32(sV + s * HEAD_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < BN / 16; ++k) {
                    const uint32_t a_off = (k >> 2) * HALF_BYTES + (k & 3) * 32;    // P: K-major over the keys
                    const uint32_t b_off = (uint32_t)k * 16 * 128;                  // V: 16 key rows of 128 bytes further
                    umma_bf16(tmem_base + 256 + b * HD, smem_desc_sw128(p_addr + a_off, 16, 1024), smem_desc_sw128(v_addr + b_off, HALF_BYTES, 1024), IDESC_PV, (u | (uint32_t)k) ? 1u : 0u);
                }
                umma_commit(smem_u32(&ctl->pv_done[b]));
                umma_commit(smem_u32(&ctl->v_empty[s]));
            }
        }
    } else {
        // ---- softmax and output: group g (warps 2 + 4g .. 5 + 4g) takes the key tiles of parity g, one thread per row ----
        // Warp w may read tensor-memory lanes 32*(w%4)..+31.
        const int q = warp & 3;
        const uint32_t g = (uint32_t)(warp - 2) >> 2;
        const int row = q * 32 + lane;
        const int pos = pos0 + row;
        const bool row_valid = row < n_rows;
        const int wlo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        const uint32_t s_addr = lane_addr + g * 128, o_addr = lane_addr + 256 + g * HD;
        float m_ref = -INFINITY;           // the maximum the group's probabilities (and its O) are taken relative to
        float l = 0.0f;                    // the group's sum for this row, relative to m_ref
        const int n_tiles_k = kt_end - kt_begin;
        uint32_t done = 0;                 // tiles of this group so far
        bool ok = true;
        uint32_t sreg[128];
        for (uint32_t it = g; (int)it < n_tiles_k && ok; it += 2, ++done) {
            const int kt = kt_begin + (int)it;
            const uint32_t u = it >> 1;
            if (!mbar_wait(smem_u32(&ctl->s_full[g]), u & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld32_nowait(s_addr + c * 32, sreg + c * 32);
            tmem_ld_wait();
            tc_fence_before();
            warp_arrive(smem_u32(&ctl->s_free[g]), lane);  // S of this tile is in registers
            const int key0 = kt * BN;
            // a tile every key of which this row sees needs no mask
            const bool interior = row_valid && key0 + BN - 1 <= pos && key0 >= wlo;
            float mx = -INFINITY;
            if (interior) {
#pragma unroll
                for (int i = 0; i < BN; ++i) mx = fmaxf(mx, __uint_as_float(sreg[i]));
            } else {
#pragma unroll
                for (int i = 0; i < BN; ++i) {
                    const int key = key0 + i;
                    if (!(row_valid && key <= pos && key >= wlo)) sreg[i] = 0xff800000u;      // -inf
                    mx = fmaxf(mx, __uint_as_float(sreg[i]));
                }
            }
            // P V of the group's previous tile is done: its P buffer is free and its O is at rest until this tile's P
            // is published
            if (done >= 1 && !mbar_wait(smem_u32(&ctl->pv_done[g]), (u - 1) & 1, abort_flag)) { ok = false; break; }
            // Move the reference only when the maximum has outgrown it by RESCALE_STEP (or there was none).  O of a
            // row without a reference is still zero.
            const bool move = mx > m_ref && (m_ref == -INFINITY || (mx - m_ref) * scale_log2 > RESCALE_STEP);
            const bool scale_o = move && m_ref != -INFINITY;
            if (__any_sync(0xffffffffu, scale_o)) {
                tc_fence_after();
                const float alpha = scale_o ? fast_exp2((m_ref - mx) * scale_log2) : 1.0f;
#pragma unroll 1
                for (int c = 0; c < HD / 16; ++c) {
                    uint32_t oreg[16];
                    tmem_ld16(o_addr + c * 16, oreg);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
                    tmem_st16(o_addr + c * 16, oreg);
                }
                tmem_st_wait();
                l *= alpha;
            }
            if (move) m_ref = mx;
            const float use = (m_ref == -INFINITY) ? 0.0f : m_ref * scale_log2;
            // probabilities, rounded to bf16 as the tensor core will read them: the row of P is two halves of 64 keys,
            // each 8 chunks of 16 bytes, chunk index xor-ed with row % 8
            float sum = 0.0f;
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                unsigned char* prow = sP + g * TILE_BYTES + hf * HALF_BYTES + row * 128;
#pragma unroll
                for (int ch = 0; ch < 8; ++ch) {
                    uint32_t packed[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float p0 = fast_exp2(fmaf(__uint_as_float(sreg[hf * 64 + ch * 8 + 2 * i]), scale_log2, -use));
                        const float p1 = fast_exp2(fmaf(__uint_as_float(sreg[hf * 64 + ch * 8 + 2 * i + 1]), scale_log2, -use));
                        sum += p0 + p1;
                        packed[i] = pack_bf16x2(p0, p1);
                    }
                    *reinterpret_cast<uint4*>(prow + ((ch ^ (row & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                }
            }
            l += sum;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // P is read by the tensor core (async proxy)
            tc_fence_before();                                                // ... and O, if it was rescaled, is in tensor memory
            warp_arrive(smem_u32(&ctl->p_full[g]), lane);
        }
        // Merge the two groups: every thread posts its row's (reference, sum); the row's output is
        // (O0 f0 + O1 f1) / (l0 f0 + l1 f1) with f = 2^((m_g - m) scale); group g writes its half of the output columns.
        ctl->xchg[g][0][row] = m_ref;
        ctl->xchg[g][1][row] = l;
        warp_arrive(smem_u32(&ctl->l_full), lane);
        if (ok) ok = mbar_wait(smem_u32(&ctl->l_full), 0, abort_flag);
        const float m0 = ctl->xchg[0][0][row], m1 = ctl->xchg[1][0][row];
        const float l0 = ctl->xchg[0][1][row], l1 = ctl->xchg[1][1][row];
        const float m = fmaxf(m0, m1);
        const float f0 = (m0 == -INFINITY) ? 0.0f : fast_exp2((m0 - m) * scale_log2);
        const float f1 = (m1 == -INFINITY) ? 0.0f : fast_exp2((m1 - m) * scale_log2);
        const float total = l0 * f0 + l1 * f1;
        // O of both groups is complete when their last P V is done (a group without tiles has no O)
        const int tiles0 = (n_tiles_k + 1) / 2, tiles1 = n_tiles_k / 2;
        if (ok && tiles0 > 0) ok = mbar_wait(smem_u32(&ctl->pv_done[0]), (uint32_t)(tiles0 - 1) & 1, abort_flag);
        if (ok && tiles1 > 0) ok = mbar_wait(smem_u32(&ctl->pv_done[1]), (uint32_t)(tiles1 - 1) & 1, abort_flag);
        tc_fence_after();
        const float inv = total > 0.0f ? 1.0f / total : 0.0f;
        __nv_bfloat16* orow = out + ((size_t)(row0 + row) * H + h) * HD + g * (HD / 2);
#pragma unroll 1
        for (int c = 0; c < HD / 64; ++c) {                        // 32 output columns at a time
            float acc[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0.0f;
            if (ok && tiles0 > 0) {                                // uniform over the CTA
                tmem_ld32_nowait(lane_addr + 256 + g * (HD / 2) + c * 32, sreg);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[i] = __uint_as_float(sreg[i]) * f0;
            }
            if (ok && tiles1 > 0) {
                tmem_ld32_nowait(lane_addr + 256 + HD + g * (HD / 2) + c * 32, sreg);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[i] = fmaf(__uint_as_float(sreg[i]), f1, acc[i]);
            }
            if (ok && row_valid) {
#pragma unroll
                for (int i = 0; i < 32; i += 8)
                    *reinterpret_cast<uint4*>(orow + c * 32 + i) = make_uint4(pack_bf16x2(acc[i] * inv, acc[i + 1] * inv), pack_bf16x2(acc[i + 2] * inv, acc[i + 3] * inv),
                                                                              pack_bf16x2(acc[i + 4] * inv, acc[i + 5] * inv), pack_bf16x2(acc[i + 6] * inv, acc[i + 7] * inv));
            }
        }
    }

    // ---- teardown ----
    if (*abort_flag) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (threadIdx.x == 0 && ctl->abort_flag && err != nullptr) atomicExch(err, 2);
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS_ATT) : "memory");
    }
}

}  // namespace

// q, out: [n_tokens, H*hd] bf16; k_pages, v_pages: [num_pages, G, page_size, hd] bf16 of one layer (hd 64 or 128);
// tiles: int32 [n_tiles, 4] (request, first row, rows <= 128, first position).  `err`: device int set to 2 when a
// bounded wait ran out (may be null).
MM_EXPORT int mm_attention_prefill_tcgen05(const void* q, const void* k_pages, const void* v_pages, void* out,
                                           const void* tiles, int n_tiles, const void* block_table, int table_width,
                                           int page_size, int num_pages, int n_tokens, int H, int G, int hd, int window,
                                           float scale, void* err, void* stream) {
    MM_REQUIRE(hd == 128 || hd == 64, "attention_prefill_tcgen05: built for head sizes 64 and 128");
    MM_REQUIRE(n_tiles >= 0 && H > 0 && G > 0 && H % G == 0 && n_tokens > 0 && num_pages > 0, "attention_prefill_tcgen05: bad sizes");
    MM_REQUIRE(page_size >= 8 && page_size <= 128 && (128 % page_size) == 0, "attention_prefill_tcgen05: page_size must be 8, 16, 32, 64 or 128");
    MM_REQUIRE(table_width > 0 && window >= 0, "attention_prefill_tcgen05: bad table or window");
    if (n_tiles == 0) return MM_OK;
    CUtensorMap tq, tk, tv;
    const long long pool_rows = (long long)num_pages * G * page_size;
    if (!tc::make_map_bf16(&tq, q, n_tokens, H * hd, (long long)H * hd, 128) ||
        !tc::make_map_bf16(&tk, k_pages, pool_rows, hd, hd, page_size) ||
        !tc::make_map_bf16(&tv, v_pages, pool_rows, hd, hd, page_size)) {
        mm_set_last_error("attention_prefill_tcgen05: cuTensorMapEncodeTiled failed or is not available");
        return MM_ERR_DRIVER;
    }
    const int halves = hd / 64;
    const size_t smem = (size_t)(halves + 4 + 2 * KV_STAGES * halves) * HALF_BYTES + sizeof(AttCtl);
    static bool configured[2] = {false, false};
    if (!configured[halves - 1]) {
        const cudaError_t e = hd == 128 ? cudaFuncSetAttribute(attention_prefill_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                                        : cudaFuncSetAttribute(attention_prefill_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            mm_set_last_error("attention_prefill_tcgen05: cannot reserve shared memory");
            return MM_ERR_LAUNCH;
        }
        configured[halves - 1] = true;
    }
    const float LOG2E = 1.4426950408889634f;
    MM_REQUIRE(n_tiles <= 65535, "attention_prefill_tcgen05: more than 65535 tiles in one launch");
    dim3 grid(H, n_tiles);
    if (hd == 128)
        attention_prefill_tc_kernel<128><<<grid, ATT_TC_THREADS, smem, (cudaStream_t)stream>>>(
            tq, tk, tv, (__nv_bfloat16*)out, (const int32_t*)tiles, (const int32_t*)block_table, table_width, page_size, H, G,
            window, scale * LOG2E, (int*)err);
    else
        attention_prefill_tc_kernel<64><<<grid, ATT_TC_THREADS, smem, (cudaStream_t)stream>>>(
            tq, tk, tv, (__nv_bfloat16*)out, (const int32_t*)tiles, (const int32_t*)block_table, table_width, page_size, H, G,
            window, scale * LOG2E, (int*)err);
    MM_CHECK_LAUNCH();
    return MM_OK;
}
