// Stage 2, primary path: BitLinear decode (M <= 16 tokens) as a weight stream through shared memory.
//
// A decode-time linear reads every packed weight byte exactly once and does almost no arithmetic
// per byte, so what matters is how many bytes are in flight per SM and how little each warp has
// to wait for anybody else.  Loads staged in registers cap the bytes in flight at (resident
// threads) x (loads per thread); here the copy engine fills shared-memory stages instead.
//
//   One persistent CTA per SM with 16 warps in `groups` groups of G = 16/groups warps (the host
//   picks G from the number of row blocks per CTA: G = 1 when every warp can have its own blocks,
//   larger when there are few blocks and a block's K range has to be split to keep all warps busy).
//   A group owns blocks of 16 consecutive output rows and a private ring of D stages of 16 rows x
//   cb packed bytes.  The group's first warp issues the copies itself -- ONE cp.async.bulk.tensor
//   per stage (2-D box, no multicast; rows past N and bytes past the row end are zero-filled),
//   D stages ahead -- so with G = 1 a warp never synchronises with another warp after start-up.
//   (One plain bulk copy per weight row, 800 bytes each, ran no faster than register-staged
//   loads: the copy engine's rate of small copies set the pace.)
//
//   A stage holds cb/64 units of 16 rows x 64 bytes (256 k).  The group's warps take units
//   round-robin, read packed words from the stage and the int8 activations from a CTA-resident
//   copy, and run the AND-only extraction + mma.sync.m16n8k32.u8.s8 of ternary_mma.cuh.  At the
//   end of a row block the other warps of the group hand their partial sums to the first one,
//   which subtracts the token's row sum (code = trit + 1), applies ((scale/127)*acc)*weight_scale
//   with separately rounded steps and stores.
//
// The activations are either given already quantised (q in consumption order + scale + rowsum),
// or (M <= 8) as fp32/fp16/bf16 rows that every CTA quantises itself while its first weight
// stages are in flight -- then a decode-time linear is one launch.  Either way they are laid out
// in shared memory with the 16-byte slots of a 64-byte group XOR-swizzled so that the B-operand
// reads of a quarter-warp fall into eight different bank groups.
//
// Every mbarrier wait is bounded in time; on expiry the kernel records a status word and the warp
// falls through to the end, after waiting (bounded) for its own copies in flight.
#include <type_traits>

#include "sm100_common.cuh"
#include "ternary_mma.cuh"

namespace nslq {

namespace stream {

using namespace sm100;

constexpr int NW = 16;                      // warps per CTA
constexpr int THREADS = NW * 32;
constexpr int ROWS = 16;                    // output rows per block = MMA M
constexpr int MAX_STAGES = 64;              // over all groups
constexpr int CB_MAX = 1024;                // packed bytes per row and stage (256 32-bit elements: the widest box)
constexpr int MAX_M = 16;
constexpr int FUSED_MAX_M = 8;

struct Params {
    const uint8_t *w;        // [N][K/4]
    const void *x;           // [M][K] fp32/fp16/bf16 (fused quantisation) or null
    const int8_t *q;         // [M][K] consumption order, when x is null
    const float *scale;      // [M], when x is null
    const int32_t *rowsum;   // [M], when x is null
    void *y;                 // [M][N]
    int32_t *acc_out;        // [M][N] or null
    const float *bias;       // [N] or null
    const float *residual;   // [M][N] or null
    int64_t N, K;
    int M, y_dtype;
    float weight_scale;
    int row_bytes, nchunk, cb, kp;
    int G, groups, D;                           // warps per group, groups, stages per group
    int off_misc, off_red, off_ring, off_bar;   // shared-memory map (bytes)
};

// physical 32-bit word of activation word v (v = k/4 in consumption order) inside a token row
static __device__ __forceinline__ int act_word(int v)
{
    const int slot = v >> 2, c = slot >> 2, j = slot & 3;
    return (((c << 2) | (j ^ ((c >> 1) & 3))) << 2) | (v & 3);
}

// One token row: absmax, the reference's rounding and the row sum, by the threads `tid` of `nthr`
// (whole warps).  Returns this thread's partial row sum; `scale` is the row's absmax.
template <typename XT>
static __device__ __forceinline__ int quantise_row(const XT *xr, uint32_t *q_row, int nvec, float scale, int tid, int nthr)
{
    const float inv = __fdiv_rn(127.0f, scale);
    const bool zero_row = (scale == 0.0f);
    int sum = 0;
    for (int base = 0; base < nvec; base += nthr) {
        const int v = base + tid;
        const bool in = v < nvec;
        const unsigned mask = __ballot_sync(0xffffffffu, in);     // whole quads: K % 64 == 0
        if (in) {
            const float4 f = Vec4<XT>::load(xr, v);
            const int q0 = zero_row ? 0 : quant_one(f.x, inv), q1 = zero_row ? 0 : quant_one(f.y, inv);
            const int q2 = zero_row ? 0 : quant_one(f.z, inv), q3 = zero_row ? 0 : quant_one(f.w, inv);
            sum += q0 + q1 + q2 + q3;
            q_row[act_word(v)] = quad_transpose(pack4_i8(q0, q1, q2, q3), mask);
        }
    }
    return sum;
}
template <typename XT>
static __device__ __forceinline__ float absmax_row(const XT *xr, int nvec, int tid, int nthr)
{
    float mx = 0.0f;
    int v = tid;
    for (; v + 3 * nthr < nvec; v += 4 * nthr) {                    // four loads in flight per lane
        float4 f[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = Vec4<XT>::load(xr, v + i * nthr);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(f[i].x), fabsf(f[i].y)), fmaxf(fabsf(f[i].z), fabsf(f[i].w))));
    }
    for (; v < nvec; v += nthr) {
        const float4 f = Vec4<XT>::load(xr, v);
        mx = fmaxf(mx, fmaxf(fmaxf(fabsf(f.x), fabsf(f.y)), fmaxf(fabsf(f.z), fabsf(f.w))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    return mx;
}

template <int NT, typename XT>
__global__ void __launch_bounds__(THREADS, 1)
ternary_stream_kernel(const __grid_constant__ CUtensorMap tmap_w, const Params p)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // misc block: zero[64 B] scale_s[16] rowsum_s[16] part_f[NW][2] part_i[NW][2]
    uint8_t *zero_blk = smem + p.off_misc;
    float *scale_s = reinterpret_cast<float *>(zero_blk + 64);
    int *rowsum_s = reinterpret_cast<int *>(scale_s + MAX_M);
    float *part_f = reinterpret_cast<float *>(rowsum_s + MAX_M);
    int *part_i = reinterpret_cast<int *>(part_f + NW * 2);
    int *red = reinterpret_cast<int *>(smem + p.off_red);            // [NW][NT*4][32]
    const uint32_t bars = sbase + p.off_bar;
    // barriers: full[groups*D] (copy landed), empty[groups*D] (the group's other warps are done with
    // the stage), redf[groups] (their partial sums are written), rede[groups] (and read again)
    const int nst = p.groups * p.D;
    auto full_bar = [&](int i) { return bars + 8u * i; };
    auto empty_bar = [&](int i) { return bars + 8u * (MAX_STAGES + i); };
    auto redf_bar = [&](int gi) { return bars + 8u * (2 * MAX_STAGES + gi); };
    auto rede_bar = [&](int gi) { return bars + 8u * (2 * MAX_STAGES + NW + gi); };

    const int gi = warp / p.G, wg = warp % p.G;                      // group, warp within the group
    const bool head = (wg == 0);
    const int nblocks = (int)((p.N + ROWS - 1) / ROWS);
    const int stage_bytes = ROWS * p.cb;                             // the copy engine writes the box densely
    const uint32_t ring = sbase + p.off_ring + (uint32_t)(gi * p.D) * stage_bytes;
    const uint8_t *ring_ptr = smem + p.off_ring + (size_t)(gi * p.D) * stage_bytes;
    // this group's work: the CTA's blocks j = gi, gi + groups, ...; `total` stages in all
    const int cta_blocks = blockIdx.x < nblocks ? (nblocks - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int my_blocks = gi < cta_blocks ? (cta_blocks - 1 - gi) / p.groups + 1 : 0;
    const int total = my_blocks * p.nchunk;
    auto stage_block = [&](int i) { return (int)blockIdx.x + (gi + (i / p.nchunk) * p.groups) * (int)gridDim.x; };

    if (threadIdx.x == 0) {
        for (int i = 0; i < nst; ++i) { mbar_init(full_bar(i), 1); mbar_init(empty_bar(i), p.G > 1 ? p.G - 1 : 1); }
        for (int i = 0; i < p.groups; ++i) { mbar_init(redf_bar(i), p.G > 1 ? p.G - 1 : 1); mbar_init(rede_bar(i), 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // The weights do not depend on the preceding kernel of the stream: start the first D stages
    // of every group before waiting for it, and let the next kernel do the same.
    auto issue = [&](int i) {                                        // stage use i of this group
        const int sl = i % p.D;
        mbar_arrive_expect_tx(full_bar(gi * p.D + sl), (uint32_t)stage_bytes);   // a box counts in full, filled part included
        tma_load_2d(ring + sl * stage_bytes, &tmap_w, (i % p.nchunk) * (p.cb >> 2), stage_block(i) * ROWS, full_bar(gi * p.D + sl));
    };
    int issued = p.D < total ? p.D : total;
    if (head && lane == 0)
        for (int i = 0; i < issued; ++i) issue(i);
    pdl_launch_dependents();
    pdl_wait();

    // ---------------- activations into shared memory (all warps)
    if (threadIdx.x < 16) reinterpret_cast<uint32_t *>(zero_blk)[threadIdx.x] = 0u;
    if constexpr (std::is_void<XT>::value) {
        const int slots = (int)(p.K >> 4), all = slots * p.M;
        const uint4 *src = reinterpret_cast<const uint4 *>(p.q);        // rows are contiguous: [M][K]
#pragma unroll 4
        for (int e = threadIdx.x; e < all; e += THREADS) {
            const int m = e / slots, sl = e - m * slots;
            const int c = sl >> 2, j = sl & 3;
            reinterpret_cast<uint4 *>(smem + (size_t)m * p.kp)[(c << 2) | (j ^ ((c >> 1) & 3))] = __ldg(src + e);
        }
        if (threadIdx.x < p.M) { scale_s[threadIdx.x] = p.scale[threadIdx.x]; rowsum_s[threadIdx.x] = p.rowsum[threadIdx.x]; }
    } else {
        // same arithmetic as act_quant_kernel.  The 16 warps are dealt out to the tokens (16, 8, 4
        // or 2 warps each), so the rows run side by side with several loads in flight per lane.
        const XT *x = reinterpret_cast<const XT *>(p.x);
        const int nvec = (int)(p.K >> 2);
        const int wpt = p.M <= 1 ? 16 : (p.M <= 2 ? 8 : (p.M <= 4 ? 4 : 2));   // warps per token
        const int m = warp / wpt, tid = (warp % wpt) * 32 + lane, nthr = wpt * 32;
        const bool live = m < p.M;
        if (live) {
            const float mx = absmax_row(x + (int64_t)m * p.K, nvec, tid, nthr);
            if (lane == 0) part_f[warp] = mx;
        }
        __syncthreads();
        if (live) {
            float scale = 0.0f;
            for (int w = 0; w < wpt; ++w) scale = fmaxf(scale, part_f[m * wpt + w]);
            int sum = quantise_row(x + (int64_t)m * p.K, reinterpret_cast<uint32_t *>(smem + (size_t)m * p.kp), nvec, scale, tid, nthr);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (lane == 0) part_i[warp] = sum;
            if (tid == 0) scale_s[m] = scale;
        }
        __syncthreads();
        if (threadIdx.x < p.M) {
            int tot = 0;
            for (int w = 0; w < wpt; ++w) tot += part_i[threadIdx.x * wpt + w];
            rowsum_s[threadIdx.x] = tot;
        }
    }
    __syncthreads();

    // ---------------- stream this group's stages
    const int g = lane >> 2, t = lane & 3;
    // Shared-memory bandwidth is what this loop runs into (a unit of 1 KiB of weights is written
    // once by the copy engine and read once, 16 wavefronts, and every 8-token B fragment set is
    // another 16), so lanes whose token does not exist issue no load at all: a 128-bit load costs
    // one wavefront per quarter-warp that has an active lane.
    const uint8_t *qbase[NT];
    bool tok_ok[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int tok = nt * 8 + g;
        tok_ok[nt] = tok < p.M;
        qbase[nt] = smem + (size_t)(tok_ok[nt] ? tok : 0) * p.kp;
    }
    // independent MMA chains per warp: 4 position classes x NA word pairs x NT token tiles = 8
    constexpr int NA = (NT == 1) ? 2 : 1;
    Acc4 acc[NT][NA];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int k = 0; k < NA; ++k) acc_zero(acc[nt][k]);
    const int nchunks16 = (int)(p.K >> 6);
    bool ok = true;
    int c = 0;                                                       // chunk of the current block
    for (int i = 0; i < total && ok; ++i) {
        const int sl = i % p.D;
        const uint32_t ph = (uint32_t)(i / p.D) & 1u;
        if (!(ok = mbar_wait(full_bar(gi * p.D + sl), ph, 0x511))) break;
        const uint8_t *st = ring_ptr + (size_t)sl * stage_bytes;
        const int bytes = c == p.nchunk - 1 ? p.row_bytes - c * p.cb : p.cb;
        const int units = (bytes + 63) >> 6, ubase = (c * p.cb) >> 6;
#pragma unroll 2
        for (int u = (wg + i) % p.G; u < units; u += p.G) {           // rotate so that odd unit counts even out
            const int ug = ubase + u, c16 = 4 * ug + t;
            const bool in = c16 < nchunks16;                          // the row may end inside the unit
            uint4 ra = *reinterpret_cast<const uint4 *>(st + g * p.cb + 64 * u + 16 * t);
            uint4 rb = *reinterpret_cast<const uint4 *>(st + (g + 8) * p.cb + 64 * u + 16 * t);
            if (!in) { ra = make_uint4(0, 0, 0, 0); rb = ra; }        // code 0 contributes nothing
            const int f = ((ug & 1) << 1) | (t >> 1);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                uint4 xq[4];
                const uint8_t *qp = qbase[nt] + (size_t)c16 * 64;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    xq[j] = tok_ok[nt] ? *reinterpret_cast<const uint4 *>(qp + ((j ^ f) << 4)) : make_uint4(0, 0, 0, 0);
                if constexpr (NA == 2) chunk_mma2(acc[nt][0], acc[nt][1], ra, rb, xq);
                else chunk_mma(acc[nt][0], ra, rb, xq);
            }
        }
        // give the stage back and refill it D uses ahead
        __syncwarp();
        if (head) {
            if (p.G > 1 && !(ok = mbar_wait(empty_bar(gi * p.D + sl), ph, 0x512))) break;
            if (lane == 0 && issued < total) { issue(issued); }
            ++issued;
        } else if (lane == 0) {
            mbar_arrive(empty_bar(gi * p.D + sl));
        }
        if (++c < p.nchunk) continue;
        c = 0;
        // ---- end of a row block: collect the group's partial sums in its first warp and store
        const uint32_t bph = (uint32_t)(i / p.nchunk) & 1u;
        int a[NT * 4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                int v = 0;
#pragma unroll
                for (int k = 0; k < NA; ++k) v += acc_value(acc[nt][k], r);
                a[nt * 4 + r] = v;
            }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int k = 0; k < NA; ++k) acc_zero(acc[nt][k]);
        if (p.G > 1) {
            if (!head) {
                if (!(ok = mbar_wait(rede_bar(gi), bph ^ 1u, 0x513))) break;   // the previous block's partials were read
                int *dst = red + (warp * NT * 4) * 32 + lane;
#pragma unroll
                for (int k = 0; k < NT * 4; ++k) dst[k * 32] = a[k];
                __syncwarp();
                if (lane == 0) mbar_arrive(redf_bar(gi));
                continue;
            }
            if (!(ok = mbar_wait(redf_bar(gi), bph, 0x514))) break;
            for (int w = 1; w < p.G; ++w) {
                const int *src = red + ((gi * p.G + w) * NT * 4) * 32 + lane;
#pragma unroll
                for (int k = 0; k < NT * 4; ++k) a[k] += src[k * 32];
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(rede_bar(gi));
        }
        // C fragment of m16n8: registers 0,1 = row g, tokens 2t, 2t+1; registers 2,3 = row g+8
        const int blk = stage_block(i);
#pragma unroll
        for (int k = 0; k < NT * 4; ++k) {
            const int nt = k >> 2, r = k & 3;
            const int tok = nt * 8 + 2 * t + (r & 1);
            const int64_t n = (int64_t)blk * ROWS + g + 8 * (r >> 1);
            if (tok < p.M && n < p.N) {
                const int accv = a[k] - rowsum_s[tok];
                const int64_t o = (int64_t)tok * p.N + n;
                if (p.acc_out) p.acc_out[o] = accv;
                float v = bitlinear_finalize(accv, scale_s[tok], p.weight_scale);
                if (p.bias) v = __fadd_rn(v, p.bias[n]);
                if (p.residual) v = __fadd_rn(v, p.residual[o]);
                store_out(p.y, p.y_dtype, o, v);
            }
        }
    }
    if (!ok && head && lane == 0) {
        // gave up somewhere: let this group's copies already issued land before the CTA retires
        const int n = issued < p.D ? issued : p.D;
        for (int k = 0; k < n; ++k) {
            const int idx = (issued < total ? issued : total) - 1 - k;
            if (idx >= 0) (void)mbar_wait(full_bar(gi * p.D + idx % p.D), (uint32_t)(idx / p.D) & 1u, 0x515);
        }
    }
}

}  // namespace stream

// ---------------------------------------------------------------- host side
static int smem_budget()
{
    static int v = 0;
    if (!v) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    }
    return v;
}

// Fills the geometry fields; false when the shape does not fit (too few stages would be left).
static bool plan(stream::Params &p, int NT, int *smem_bytes, int *grid_out)
{
    using namespace stream;
    p.row_bytes = (int)(p.K >> 2);
    const int nblocks = (int)((p.N + ROWS - 1) / ROWS);
    const int grid = nblocks < sm100::sm_count() ? nblocks : sm100::sm_count();
    // warps per group: every warp on its own when a CTA has at least NW row blocks, otherwise
    // the K range of a block is split over G warps so that none is idle
    const int bpc = (nblocks + grid - 1) / grid;
    p.groups = 1;
    while (p.groups < bpc && p.groups < NW) p.groups <<= 1;
    p.G = NW / p.groups;
    p.kp = (int)(((p.K + 127) / 128) * 128 + 32);                   // = 32 mod 128: two tokens of a quarter-warp in different banks
    const int act = (p.M * p.kp + 127) & ~127;
    const int misc = 64 + MAX_M * 8 + NW * 2 * 8;
    const int red = NW * NT * 4 * 32 * 4;
    p.off_misc = act;
    p.off_red = (p.off_misc + misc + 127) & ~127;
    p.off_ring = (p.off_red + red + 1023) & ~1023;
    const int bar_bytes = (2 * MAX_STAGES + 2 * NW) * 8;
    const int room = smem_budget() - p.off_ring - bar_bytes - 128;
    if (room <= 0) return false;
    int cb_cap = (room / (p.groups * 2 * ROWS)) & ~63;              // at least two stages per group
    if (cb_cap > CB_MAX) cb_cap = CB_MAX;
    if (cb_cap < 64) return false;
    int nchunk = (p.row_bytes + cb_cap - 1) / cb_cap;
    p.cb = (((p.row_bytes + nchunk - 1) / nchunk) + 63) & ~63;      // even split, whole 64-byte units
    // rows of a stage lie cb apart: an odd multiple of 64 keeps the 128-bit reads of two rows in
    // different banks
    if ((p.cb & 64) == 0) { if (p.cb + 64 <= cb_cap) p.cb += 64; else if (p.cb > 64) p.cb -= 64; }
    p.nchunk = (p.row_bytes + p.cb - 1) / p.cb;
    p.D = room / (p.groups * ROWS * p.cb);
    if (p.D > 4) p.D = 4;
    if (p.D < 2) return false;
    p.off_bar = p.off_ring + p.groups * p.D * ROWS * p.cb;
    *smem_bytes = p.off_bar + bar_bytes;
    *grid_out = grid;
    return true;
}

// The packed weight as a 2-D tensor of 32-bit words (a box may be 256 elements wide: 1024 bytes).
static int make_weight_map(CUtensorMap *m, const stream::Params &p)
{
    sm100::EncodeTiledFn enc = sm100::encode_tiled();
    if (!enc) return fail(NSLQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t gdim[2] = {(cuuint64_t)(p.row_bytes >> 2), (cuuint64_t)p.N};
    const cuuint64_t gstride[1] = {(cuuint64_t)p.row_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)(p.cb >> 2), (cuuint32_t)stream::ROWS};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t *>(p.w), gdim, gstride, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(NSLQ_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for the packed weight %lld x %d bytes", (int)r,
                    (long long)p.N, p.row_bytes);
    return NSLQ_OK;
}

template <int NT, typename XT>
static int launch_stream(const stream::Params &p, int smem, int grid, cudaStream_t st)
{
    static int reserved = 0;
    if (smem > reserved) {
        if (cudaFuncSetAttribute(stream::ternary_stream_kernel<NT, XT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return fail(NSLQ_ERR_CUDA, "ternary_stream_kernel: cannot reserve %d bytes of shared memory: %s", smem,
                        cudaGetErrorString(cudaGetLastError()));
        reserved = smem;
    }
    CUtensorMap tmap_w;
    int rc = make_weight_map(&tmap_w, p);
    if (rc) return rc;
    cudaError_t e = launch_kernel(stream::ternary_stream_kernel<NT, XT>, dim3(grid), dim3(stream::THREADS), (size_t)smem, st, tmap_w, p);
    if (e != cudaSuccess) return fail(NSLQ_ERR_CUDA, "ternary_stream_kernel: %s", cudaGetErrorString(e));
    return check_launch("ternary_stream_kernel");
}

static bool stream_shape_ok(const void *w, int64_t M, int64_t N, int64_t K)
{
    return M >= 1 && M <= stream::MAX_M && (K % 64 == 0) && aligned16(w) && N < (1ll << 31) && K < (1ll << 28);
}

// Already-quantised activations (consumption order), M <= 16.
bool ternary_stream_supported(const void *w, const void *q_perm, int64_t M, int64_t N, int64_t K)
{
    if (!stream_shape_ok(w, M, N, K) || !aligned16(q_perm)) return false;
    stream::Params p{};
    p.N = N; p.K = K; p.M = (int)M;
    int smem = 0, grid = 0;
    return plan(p, M <= 8 ? 1 : 2, &smem, &grid);
}

int ternary_stream_dispatch(const uint8_t *w, const int8_t *q_perm, const float *scale, const int32_t *rowsum, int M,
                            int64_t N, int64_t K, float weight_scale, void *y, int y_dtype, int32_t *acc_out,
                            const float *bias, const float *residual, cudaStream_t st)
{
    stream::Params p{};
    p.w = w; p.q = q_perm; p.scale = scale; p.rowsum = rowsum; p.y = y; p.acc_out = acc_out; p.bias = bias;
    p.residual = residual; p.N = N; p.K = K; p.M = M; p.y_dtype = y_dtype; p.weight_scale = weight_scale;
    int smem = 0, grid = 0;
    if (!plan(p, M <= 8 ? 1 : 2, &smem, &grid)) return fail(NSLQ_ERR_UNSUPPORTED, "ternary_stream_kernel: M=%d K=%lld does not fit shared memory", M, (long long)K);
    return M <= 8 ? launch_stream<1, void>(p, smem, grid, st) : launch_stream<2, void>(p, smem, grid, st);
}

// Activations in their own dtype, quantised inside the kernel; M <= 8.
bool ternary_stream_fused_supported(const void *w, const void *x, int x_dtype, int64_t M, int64_t N, int64_t K)
{
    if (!stream_shape_ok(w, M, N, K) || M > stream::FUSED_MAX_M || !aligned16(x)) return false;
    if (x_dtype != NSLQ_DTYPE_F32 && x_dtype != NSLQ_DTYPE_FP16 && x_dtype != NSLQ_DTYPE_BF16) return false;
    stream::Params p{};
    p.N = N; p.K = K; p.M = (int)M;
    int smem = 0, grid = 0;
    return plan(p, 1, &smem, &grid);
}

int ternary_stream_fused_dispatch(const uint8_t *w, const void *x, int x_dtype, int M, int64_t N, int64_t K,
                                  float weight_scale, void *y, int y_dtype, int32_t *acc_out, const float *bias,
                                  const float *residual, cudaStream_t st)
{
    stream::Params p{};
    p.w = w; p.x = x; p.y = y; p.acc_out = acc_out; p.bias = bias; p.residual = residual;
    p.N = N; p.K = K; p.M = M; p.y_dtype = y_dtype; p.weight_scale = weight_scale;
    int smem = 0, grid = 0;
    if (!plan(p, 1, &smem, &grid)) return fail(NSLQ_ERR_UNSUPPORTED, "ternary_stream_kernel: M=%d K=%lld does not fit shared memory", M, (long long)K);
    switch (x_dtype) {
    case NSLQ_DTYPE_F32: return launch_stream<1, float>(p, smem, grid, st);
    case NSLQ_DTYPE_FP16: return launch_stream<1, __half>(p, smem, grid, st);
    case NSLQ_DTYPE_BF16: return launch_stream<1, __nv_bfloat16>(p, smem, grid, st);
    default: return fail(NSLQ_ERR_ARG, "BitLinear: x_dtype %d not in {F32,FP16,BF16}", x_dtype);
    }
}

// The status word of this translation unit's kernels (see sm100::read_wait_status).
int ternary_stream_status(int *out) { return sm100::read_wait_status(out); }

}  // namespace nslq
