// Cross-GPU merge of sequence-sharded decode: one kernel does the local merge of this GPU's split
// partials, stores the merged (acc, m, l) record straight into every GPU's exchange buffer over
// NVLink (plain peer stores only), waits - with a bound - for the records of the other GPUs, and
// merges the `world` records.  The arithmetic is the reference's split/combine
// (crates/cuda/kernels/ops.cu:539-574) with "split" = GPU.  The reference itself is single-GPU; this
// path has no counterpart there.
//
// The records travel as 8-byte words {value, epoch}, each written and read by one 64-bit access, so a reader that
// sees the call's epoch in a word also sees its value, and no memory fence or separate flag is needed
// (a system-scope fence after peer stores costs several microseconds - more than the whole transfer).
//
// Exchange buffer of one rank (all ranks use the same layout):
//   uint2 rec[2][world][block]   block = rows*d_v accumulators, then rows*2 (m, l); the leading index
//                                is the parity of the call's epoch, so a rank that is one call ahead
//                                never overwrites a word another rank has still to read
//   uint32 ctr, done             device-kept epoch (for callers that pass epoch = 0, e.g. inside a
//                                CUDA graph, where a launch argument cannot change between replays) and
//                                the count of finished blocks that advances it at the end of a launch
// Every spin is bounded; on expiry the kernel sets bit 16 of the status word and leaves o unwritten.
#include <string.h>

#include "combine.cuh"
#include "internal.cuh"
#include "sm100_prims.cuh"

namespace gs {
namespace {

constexpr int kMaxWorld = 8;
constexpr int32_t ST_EXCHANGE = 1 << 16;

struct ExchangeLayout {
    int64_t block_words, ctr_off, total;
    int items;
};
ExchangeLayout exchange_layout(int world, int rows, int d_v) {
    ExchangeLayout L;
    L.block_words = ((int64_t) rows * (d_v + 2) + 31) / 32 * 32;  // 8-byte words, 256-byte multiple
    L.items = rows * ((d_v + CB_COLS - 1) / CB_COLS);
    L.ctr_off = 2 * (int64_t) world * L.block_words * 8;
    L.total = L.ctr_off + 256;
    return L;
}

struct ExchangeParams {
    unsigned char *bufs[kMaxWorld];  // every rank's exchange buffer, as mapped here
    int world, rank;
    uint32_t epoch;
    int64_t block_words, ctr_off;
    int rows, d_v;
    long long wait_limit;
    float *o;
    int32_t *status;
};

// One 64-bit scalar access per word (value in the low half, epoch in the high half): a scalar access of a naturally
// aligned 8-byte word is single-copy atomic, a two-element vector access is only a pair of 4-byte accesses.
__device__ __forceinline__ void st_word(uint2 *p, float v, uint32_t epoch) {
    const uint64_t w = (uint64_t) __float_as_uint(v) | ((uint64_t) epoch << 32);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ uint2 ld_word(const uint2 *p) {
    uint64_t w;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return make_uint2((uint32_t) w, (uint32_t) (w >> 32));
}

// Leaves the launch: with device-kept epochs the last block to finish advances the counter.
__device__ __forceinline__ void exchange_block_done(const ExchangeParams &X) {
    if (X.epoch != 0) return;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t *ctr = reinterpret_cast<uint32_t *>(X.bufs[X.rank] + X.ctr_off);
        const uint32_t n_blocks = gridDim.x * gridDim.y;
        if (atomicAdd(ctr + 1, 1u) == n_blocks - 1) {
            ctr[1] = 0;
            __threadfence();
            atomicAdd(ctr, 1u);
        }
    }
}

struct ExchangeLaunch {
    CUtensorMap tm;  // records as the 3-D tensor {d_v, rows, segments}; used when `tma` is set
    CombinePlan c;
    ExchangeParams x;
    int tma;
};

__global__ void __launch_bounds__(CB_NT) k_exchange_combine(const __grid_constant__ ExchangeLaunch EL) {
    const CombinePlan &C = EL.c;
    const ExchangeParams &X = EL.x;
    extern __shared__ unsigned char xraw[];
    float4 *tile = reinterpret_cast<float4 *>((reinterpret_cast<uintptr_t>(xraw) + 127) & ~(uintptr_t) 127);
    __shared__ __align__(8) uint64_t bar;
    __shared__ int s_fetch_abort;
    __shared__ CombineSmem S;
    __shared__ float s_m[kMaxWorld], s_l[kMaxWorld], s_w[kMaxWorld];
    __shared__ int s_abort;
    const int row = blockIdx.x, chunk = blockIdx.y;
    const int tid = threadIdx.x;
    if (tid == 0) {
        s_abort = 0;
        s_fetch_abort = 0;
        if (EL.tma) {
            sm100::mbar_init(&bar, 1);
            sm100::fence_barrier_init();
        }
    }
    __syncthreads();
#if __CUDA_ARCH__ >= 900
    cudaGridDependencySynchronize();  // the split partials are written by the preceding kernel
#endif
    // the epoch of this call: the caller's, or one more than the count of completed device-kept launches
    const uint32_t epoch = X.epoch ? X.epoch
                                   : *reinterpret_cast<volatile const uint32_t *>(X.bufs[X.rank] + X.ctr_off) + 1u;
    const int64_t slot = ((int64_t) (epoch & 1) * X.world) * X.block_words;  // this parity's records
    const int64_t ml_off = (int64_t) X.rows * X.d_v + (int64_t) row * 2;
    // ---- phase 1: local merge, record slice into slot [rank] of every rank's buffer ------------------
    {
        float4 a;
        float M, L;
        int col;
        const SegRange R = combine_locate(C, row, S);
        bool holds;
        if (EL.tma) {  // the item's pieces of all local segments by one tiled TMA copy
            if (!combine_item_fetch_tma(C, &EL.tm, R, chunk * CB_COLS, tile, &bar, &s_fetch_abort, S, a, M, L)) {
                exchange_block_done(X);
                return;  // status bit 18 says why; nothing is sent, the other ranks' waits run out
            }
            col = chunk * CB_COLS + (tid & 31) * 4;
            holds = tid < 32 && col < C.d_v;
            __syncthreads();  // shared memory is reused below
        } else {
            holds = combine_item_compute(C, R, chunk * CB_COLS, S, a, M, L, col);
        }
        if (holds) {
            for (int r = 0; r < X.world; r++) {
                uint2 *dst = reinterpret_cast<uint2 *>(X.bufs[r]) + slot + (int64_t) X.rank * X.block_words;
                uint2 *w = dst + (int64_t) row * X.d_v + col;
                st_word(w + 0, a.x, epoch);
                st_word(w + 1, a.y, epoch);
                st_word(w + 2, a.z, epoch);
                st_word(w + 3, a.w, epoch);
                if (col == 0) {
                    st_word(dst + ml_off, M, epoch);
                    st_word(dst + ml_off + 1, L, epoch);
                }
            }
        }
    }
    // ---- phase 2: read every rank's slice of this item; a word is there once it carries the epoch -----
    const uint2 *rec = reinterpret_cast<const uint2 *>(X.bufs[X.rank]) + slot;
    const int quad = tid % (CB_COLS / 4), sl = tid / (CB_COLS / 4);  // 32 column quads x 8 source lanes
    const int col = chunk * CB_COLS + quad * 4;
    const long long t0 = clock64();
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (sl < X.world && col < X.d_v) {
        const uint2 *w = rec + (int64_t) sl * X.block_words + (int64_t) row * X.d_v + col;
        for (;;) {
            const uint2 w0 = ld_word(w), w1 = ld_word(w + 1), w2 = ld_word(w + 2), w3 = ld_word(w + 3);
            if (w0.y == epoch && w1.y == epoch && w2.y == epoch && w3.y == epoch) {
                v = make_float4(__uint_as_float(w0.x), __uint_as_float(w1.x), __uint_as_float(w2.x), __uint_as_float(w3.x));
                break;
            }
            if (clock64() - t0 > X.wait_limit) {
                s_abort = 1;
                break;
            }
        }
    }
    if (tid < X.world) {
        const uint2 *w = rec + (int64_t) tid * X.block_words + ml_off;
        for (;;) {
            const uint2 w0 = ld_word(w), w1 = ld_word(w + 1);
            if (w0.y == epoch && w1.y == epoch) {
                s_m[tid] = __uint_as_float(w0.x);
                s_l[tid] = __uint_as_float(w1.x);
                break;
            }
            if (clock64() - t0 > X.wait_limit) {
                s_abort = 1;
                break;
            }
        }
    }
    __syncthreads();
    if (s_abort) {
        if (tid == 0) atomicOr(X.status, ST_EXCHANGE);
        exchange_block_done(X);
        return;
    }
    if (tid == 0) {
        float M = -INFINITY;
        for (int s = 0; s < X.world; s++) M = fmaxf(M, s_m[s]);
        float L = 0.f;
        for (int s = 0; s < X.world; s++) {
            const float w = s_m[s] == -INFINITY ? 0.f : expf(s_m[s] - M);
            s_w[s] = w;
            L += s_l[s] * w;
        }
        s_l[0] = L;
    }
    __syncthreads();
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (sl < X.world && s_w[sl] != 0.f) {
        const float w = s_w[sl];
        a = make_float4(v.x * w, v.y * w, v.z * w, v.w * w);
    }
    S.part[sl][quad] = a;
    __syncthreads();
    if (sl == 0 && col < X.d_v) {
#pragma unroll
        for (int j = 1; j < CB_LANES; j++) {
            const float4 u = S.part[j][quad];
            a.x += u.x;
            a.y += u.y;
            a.z += u.z;
            a.w += u.w;
        }
        const float L = s_l[0];
        const float inv = L > 0.f ? 1.f / L : 0.f;
        *reinterpret_cast<float4 *>(X.o + (int64_t) row * X.d_v + col) = make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
    }
    exchange_block_done(X);
}

}  // namespace

int launch_exchange_combine(CombinePlan c, const gs_shard_exchange &x, float *o, int32_t *status, int sm_count,
                            cudaStream_t st) {
    const int rows = c.n_seq * c.T * c.H;
    if (x.world < 2 || x.world > kMaxWorld || x.rank < 0 || x.rank >= x.world)
        return fail_invalid("exchange: world must be 2..8 and 0 <= rank < world");
    if (!x.peer_bufs || !o || !status) return fail_invalid("exchange: peer_bufs, o and a workspace are required");
    if (c.d_v % 4 != 0) return fail_invalid("exchange: d_v must be a multiple of 4");
    const ExchangeLayout L = exchange_layout(x.world, rows, c.d_v);
    if (x.buf_bytes < L.total) {
        set_error("exchange: buffers of %lld bytes needed, %lld given", (long long) L.total, (long long) x.buf_bytes);
        return (int) cudaErrorInvalidValue;
    }
    ExchangeLaunch EL;
    memset(&EL, 0, sizeof(EL));
    ExchangeParams &X = EL.x;
    for (int r = 0; r < x.world; r++) {
        if (!x.peer_bufs[r]) return fail_invalid("exchange: null peer buffer");
        X.bufs[r] = (unsigned char *) x.peer_bufs[r];
    }
    c.o = nullptr;
    c.part_out = nullptr;
    X.world = x.world;
    X.rank = x.rank;
    X.epoch = x.epoch;
    X.block_words = L.block_words;
    X.ctr_off = L.ctr_off;
    X.rows = rows;
    X.d_v = c.d_v;
    X.wait_limit = x.wait_limit_cycles > 0 ? x.wait_limit_cycles : sm100::kWaitLimitCycles;
    X.o = o;
    X.status = status;
    EL.c = c;
    // records of the tcgen05 kernel: fetched like the plain combine does, one tiled TMA copy per item
    EL.tma = c.bulk && c.desc != nullptr && c.seq_lens != nullptr && c.n_seq < 16 && c.n_ctas > 0 && c.n_ctas <= CB_NT &&
             c.d_v % CB_COLS == 0 && c.n_segments > 0 && c.seg_stride_acc % c.d_v == 0 && !(reinterpret_cast<uintptr_t>(c.acc) & 15);
    int smem = 0;
    if (EL.tma) {
        if (int e = encode_tmap_3d_f32(&EL.tm, c.acc, (uint64_t) c.d_v, (uint64_t) (c.seg_stride_acc / c.d_v), (uint64_t) c.n_segments,
                                       (uint64_t) c.d_v * 4, (uint64_t) c.seg_stride_acc * 4, CB_COLS, 1, (uint32_t) c.n_ctas))
            return e;
        smem = c.n_ctas * CB_COLS * 4 + 128;
        GS_TRY(cudaFuncSetAttribute(k_exchange_combine, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    }
    // blocks of one rank wait for blocks of the others: every block of the grid must be resident
    int per_sm = 0;
    GS_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_exchange_combine, CB_NT, smem));
    if (L.items > per_sm * sm_count && EL.tma) {  // the staging area of the tiled copy costs residency: plain loads instead
        EL.tma = 0;
        smem = 0;
        GS_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_exchange_combine, CB_NT, 0));
    }
    if (L.items > per_sm * sm_count)
        return fail_invalid("exchange: more (row, chunk) items than blocks the GPU can hold at once; use the all-gather path");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows, (c.d_v + CB_COLS - 1) / CB_COLS);
    cfg.blockDim = dim3(CB_NT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    GS_TRY(cudaLaunchKernelEx(&cfg, k_exchange_combine, EL));
    return 0;
}

}  // namespace gs

using namespace gs;

GS_EXPORT int64_t gs_shard_exchange_bytes(int world, int rows, int d_v) {
    if (world < 1 || rows < 1 || d_v < 1) return 0;
    return exchange_layout(world, rows, d_v).total;
}

GS_EXPORT int gs_peer_alloc(void **ptr, int64_t bytes) {
    if (!ptr || bytes <= 0) return fail_invalid("gs_peer_alloc: bad arguments");
    GS_TRY(cudaMalloc(ptr, (size_t) bytes));
    GS_TRY(cudaMemset(*ptr, 0, (size_t) bytes));
    GS_TRY(cudaDeviceSynchronize());
    return 0;
}
GS_EXPORT int gs_peer_free(void *ptr) {
    GS_TRY(cudaFree(ptr));
    return 0;
}
GS_EXPORT int gs_peer_export(const void *ptr, void *handle64) {
    if (!ptr || !handle64) return fail_invalid("gs_peer_export: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    GS_TRY(cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t *>(handle64), const_cast<void *>(ptr)));
    return 0;
}
GS_EXPORT int gs_peer_open(const void *handle64, void **ptr) {
    if (!ptr || !handle64) return fail_invalid("gs_peer_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    GS_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return 0;
}
GS_EXPORT int gs_peer_close(void *ptr) {
    GS_TRY(cudaIpcCloseMemHandle(ptr));
    return 0;
}
