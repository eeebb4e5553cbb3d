// Position-major export / import of a per-position cache: the bridge between a paged pool and the layout the
// reference engine saves and restores.  The reference's session state holds, for every per-position buffer of a
// layer, `unit` bytes per position for positions 0 .. upto-1, back to back (crates/engine/src/forward.rs:654-668
// position_caches, :672-681 save_state, :683-695 load_state; file format crates/engine/src/session.rs:152-204):
// the f16 latent rows, or the int8 rows and their f16 scales of a Q8 cache.  With a dense cache that is a plain
// copy of the buffer's head; with a paged pool the rows of a sequence are scattered over pages, and these two
// entry points gather them into / scatter them from exactly that byte layout, so save_state / load_state, prefix
// reuse and idle-unload parking keep working when the cache is paged.  Byte-exact: nothing is converted.
#include "internal.cuh"

namespace gs {
namespace {

constexpr int32_t ST_CACHE_IO = 1 << 19;  // status bit: a page id pointed outside the pool; that position was skipped

struct CacheIoParams {
    unsigned char *pool;       // [pool_rows][unit_bytes]
    int64_t pool_rows;
    const int32_t *pages;      // page ids of the sequence, or nullptr = dense
    int n_pages, page_rows;
    int64_t row0;              // dense: first row of the sequence
    int64_t upto;              // positions 0 .. upto-1
    int unit_bytes;
    unsigned char *flat;       // [upto][unit_bytes], position-major
    int32_t *status;           // may be nullptr
};

// One warp per position at a time (the page id is looked up once per warp), lanes over the unit's words.
template <typename W, bool IMPORT>
__global__ void __launch_bounds__(256) k_cache_io(const CacheIoParams P) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t) blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t) gridDim.x * blockDim.x) >> 5;
    const int words = P.unit_bytes / (int) sizeof(W);
    for (int64_t pos = warp; pos < P.upto; pos += n_warps) {
        int64_t row;
        if (P.pages) {
            const int64_t slot = pos / P.page_rows;
            row = slot < P.n_pages ? (int64_t) P.pages[slot] * P.page_rows + pos % P.page_rows : -1;
        } else {
            row = P.row0 + pos;
        }
        if (row < 0 || row >= P.pool_rows) {
            if (lane == 0 && P.status) atomicOr(P.status, ST_CACHE_IO);
            continue;
        }
        W *in_pool = reinterpret_cast<W *>(P.pool + row * P.unit_bytes);
        W *in_flat = reinterpret_cast<W *>(P.flat + pos * P.unit_bytes);
        for (int j = lane; j < words; j += 32) {
            if (IMPORT) in_pool[j] = in_flat[j];
            else in_flat[j] = in_pool[j];
        }
    }
}

int cache_io(bool import, const char *who, void *pool, int64_t pool_rows, const int32_t *pages, int n_pages, int page_rows,
             int64_t row0, int64_t upto, int unit_bytes, void *flat, int32_t *status, cudaStream_t st) {
    if (upto < 0 || unit_bytes <= 0 || pool_rows <= 0) {
        set_error("%s: need upto >= 0, unit_bytes > 0, pool_rows > 0", who);
        return (int) cudaErrorInvalidValue;
    }
    if (upto == 0) return 0;
    if (!pool || !flat) {
        set_error("%s: null pointer", who);
        return (int) cudaErrorInvalidValue;
    }
    if (pages && (page_rows <= 0 || n_pages <= 0 || (int64_t) n_pages * page_rows < upto)) {
        set_error("%s: the page list (%d pages of %d rows) does not cover %lld positions", who, n_pages, page_rows, (long long) upto);
        return (int) cudaErrorInvalidValue;
    }
    if (!pages && (row0 < 0 || row0 + upto > pool_rows)) {
        set_error("%s: rows %lld .. %lld lie outside the cache of %lld rows", who, (long long) row0, (long long) (row0 + upto),
                  (long long) pool_rows);
        return (int) cudaErrorInvalidValue;
    }
    CacheIoParams P{};
    P.pool = (unsigned char *) pool;
    P.pool_rows = pool_rows;
    P.pages = pages;
    P.n_pages = n_pages;
    P.page_rows = page_rows > 0 ? page_rows : 1;
    P.row0 = row0;
    P.upto = upto;
    P.unit_bytes = unit_bytes;
    P.flat = (unsigned char *) flat;
    P.status = status;
    int sms = 148;
    int dev = 0;
    GS_TRY(cudaGetDevice(&dev));
    GS_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    // HBM-bound byte work: a grid-stride loop over positions, 8 resident CTAs of 8 warps per SM
    const int64_t want = (upto + 7) / 8;
    const int grid = (int) (want < (int64_t) sms * 8 ? want : (int64_t) sms * 8);
    const uintptr_t align = reinterpret_cast<uintptr_t>(pool) | reinterpret_cast<uintptr_t>(flat) | (uintptr_t) unit_bytes;
    if ((align & 15) == 0) {
        if (import) k_cache_io<uint4, true><<<grid, 256, 0, st>>>(P);
        else k_cache_io<uint4, false><<<grid, 256, 0, st>>>(P);
    } else if ((align & 3) == 0) {
        if (import) k_cache_io<uint32_t, true><<<grid, 256, 0, st>>>(P);
        else k_cache_io<uint32_t, false><<<grid, 256, 0, st>>>(P);
    } else {
        if (import) k_cache_io<unsigned char, true><<<grid, 256, 0, st>>>(P);
        else k_cache_io<unsigned char, false><<<grid, 256, 0, st>>>(P);
    }
    GS_TRY(cudaGetLastError());
    return 0;
}

}  // namespace
}  // namespace gs

using namespace gs;

GS_EXPORT int gs_cache_export_rows(const void *pool, int64_t pool_rows, const int32_t *pages, int32_t n_pages, int32_t page_rows,
                                   int64_t row0, int64_t upto, int32_t unit_bytes, void *dst, int32_t *status, void *stream) {
    return cache_io(false, "gs_cache_export_rows", const_cast<void *>(pool), pool_rows, pages, n_pages, page_rows, row0, upto,
                    unit_bytes, dst, status, (cudaStream_t) stream);
}

GS_EXPORT int gs_cache_import_rows(void *pool, int64_t pool_rows, const int32_t *pages, int32_t n_pages, int32_t page_rows,
                                   int64_t row0, int64_t upto, int32_t unit_bytes, const void *src, int32_t *status, void *stream) {
    return cache_io(true, "gs_cache_import_rows", pool, pool_rows, pages, n_pages, page_rows, row0, upto, unit_bytes,
                    const_cast<void *>(src), status, (cudaStream_t) stream);
}
