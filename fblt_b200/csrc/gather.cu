// Batch sharding and the output gather for one process per GPU, as plain C entry points.
//
// Independent sequences are split into contiguous ranges, one per rank; nothing is exchanged
// while attention runs. Where a caller wants every rank to hold all output rows, each rank
// copies its rows into its slot of a receive buffer on every GPU: plain device-to-device
// copies through CUDA IPC mappings of the peers' buffers, which run on the copy engines over
// NVLink and take no SM from the attention launches. Nothing is ever loaded from a peer and no
// kernel waits for one; a rank's buffer is complete once every rank has passed the point the
// caller chooses (a barrier of the job, or an event per rank).
//
// The ranks find each other on the HOST, with a deadline, before the first copy is enqueued:
// fblt_rendezvous_files is an all-gather of small blobs through a directory every rank can
// reach; a rank that is absent or late is named in the error instead of leaving the others
// waiting on the device. The blobs exchanged here are the 64-byte IPC handles.
#include "common.cuh"

#include <errno.h>
#include <stdlib.h>
#include <string.h>
#include <string>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>
#include <vector>

struct fblt_gather {
    int rank, world;
    size_t max_rows, row_elems;
    float *local;              // [world, max_rows, row_elems] on this rank's GPU
    std::vector<float *> peer; // peer[r]: rank r's buffer as mapped into this process (peer[rank] == local)
    bool connected;
};

extern "C" int fblt_shard_partition(int64_t units, int32_t world, int32_t rank, int64_t *begin, int64_t *end) {
    using namespace fblt;
    if (units < 0 || world < 1 || rank < 0 || rank >= world || !begin || !end)
        return fail(FBLT_ERR_ARG, "shard_partition: bad arguments");
    // contiguous ranges, the first (units % world) ranks one unit longer
    const int64_t q = units / world, r = units % world;
    *begin = rank * q + (rank < r ? rank : r);
    *end = *begin + q + (rank < r ? 1 : 0);
    return FBLT_OK;
}

// ---- host-side rendezvous through a directory ------------------------------------------------

static double now_s() {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

static bool read_blob(const std::string &path, void *dst, size_t bytes) {
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) return false;
    const size_t n = fread(dst, 1, bytes, f);
    fclose(f);
    return n == bytes;
}

extern "C" int fblt_rendezvous_files(const char *dir, const char *tag, int32_t rank, int32_t world, const void *mine,
                                     size_t bytes, void *all, int32_t deadline_ms) {
    using namespace fblt;
    if (!dir || !tag || world < 1 || rank < 0 || rank >= world || (bytes && (!mine || !all)))
        return fail(FBLT_ERR_ARG, "rendezvous: bad arguments");
    const std::string base = std::string(dir) + "/" + tag + ".";
    // publish: write to a private name, then rename, so that a reader never sees half a blob
    {
        const std::string tmp = base + std::to_string(rank) + ".tmp", fin = base + std::to_string(rank);
        FILE *f = fopen(tmp.c_str(), "wb");
        if (!f) return fail(FBLT_ERR_ARG, "rendezvous: cannot write %s: %s", tmp.c_str(), strerror(errno));
        const size_t n = bytes ? fwrite(mine, 1, bytes, f) : 0;
        fclose(f);
        if (n != bytes || rename(tmp.c_str(), fin.c_str()) != 0)
            return fail(FBLT_ERR_ARG, "rendezvous: cannot publish %s: %s", fin.c_str(), strerror(errno));
    }
    std::vector<char> have((size_t)world, 0);
    const double t0 = now_s();
    for (;;) {
        int missing = 0, first_missing = -1;
        for (int r = 0; r < world; ++r) {
            if (have[r]) continue;
            struct stat st;
            if (stat((base + std::to_string(r) + ".failed").c_str(), &st) == 0)
                return fail(FBLT_ERR_PEER, "rendezvous '%s': rank %d announced a failure", tag, r);
            if (read_blob(base + std::to_string(r), (char *)all + (size_t)r * bytes, bytes)) {
                have[r] = 1;
            } else {
                if (first_missing < 0) first_missing = r;
                ++missing;
            }
        }
        if (!missing) return FBLT_OK;
        if ((now_s() - t0) * 1e3 >= (double)deadline_ms) {
            // say so before leaving, so that a rank arriving later does not go on alone
            FILE *f = fopen((base + std::to_string(rank) + ".failed").c_str(), "wb");
            if (f) fclose(f);
            return fail(FBLT_ERR_TIMEOUT, "rendezvous '%s': %d rank(s) did not check in within %d ms (first: rank %d)", tag,
                        missing, deadline_ms, first_missing);
        }
        usleep(2000);
    }
}

extern "C" int fblt_rendezvous_report_failure(const char *dir, const char *tag, int32_t rank) {
    using namespace fblt;
    if (!dir || !tag) return fail(FBLT_ERR_ARG, "rendezvous: bad arguments");
    const std::string path = std::string(dir) + "/" + tag + "." + std::to_string(rank) + ".failed";
    FILE *f = fopen(path.c_str(), "wb");
    if (!f) return fail(FBLT_ERR_ARG, "rendezvous: cannot write %s: %s", path.c_str(), strerror(errno));
    fclose(f);
    return FBLT_OK;
}

// ---- the gather ------------------------------------------------------------------------------

extern "C" size_t fblt_gather_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

extern "C" int fblt_gather_create(fblt_gather **out, int32_t rank, int32_t world, size_t max_rows, size_t row_elems) {
    using namespace fblt;
    if (!out || world < 1 || rank < 0 || rank >= world || max_rows == 0 || row_elems == 0)
        return fail(FBLT_ERR_ARG, "gather_create: bad arguments");
    fblt_gather *g = new fblt_gather();
    g->rank = rank;
    g->world = world;
    g->max_rows = max_rows;
    g->row_elems = row_elems;
    g->local = nullptr;
    g->connected = false;
    g->peer.assign((size_t)world, nullptr);
    const cudaError_t e = cudaMalloc(&g->local, (size_t)world * max_rows * row_elems * sizeof(float));
    if (e != cudaSuccess) {
        delete g;
        return fail(FBLT_ERR_CUDA, "gather_create: cudaMalloc: %s", cudaGetErrorString(e));
    }
    g->peer[rank] = g->local;
    *out = g;
    return FBLT_OK;
}

extern "C" int fblt_gather_export(fblt_gather *g, void *handle_out) {
    using namespace fblt;
    if (!g || !handle_out) return fail(FBLT_ERR_ARG, "gather_export: bad arguments");
    cudaIpcMemHandle_t h;
    FBLT_CUDA_TRY(cudaIpcGetMemHandle(&h, g->local));
    memcpy(handle_out, &h, sizeof(h));
    return FBLT_OK;
}

extern "C" int fblt_gather_connect(fblt_gather *g, const void *all_handles) {
    using namespace fblt;
    if (!g || !all_handles) return fail(FBLT_ERR_ARG, "gather_connect: bad arguments");
    if (g->connected) return fail(FBLT_ERR_ARG, "gather_connect: already connected");
    for (int r = 0; r < g->world; ++r) {
        if (r == g->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char *)all_handles + (size_t)r * sizeof(h), sizeof(h));
        void *p = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return fail(FBLT_ERR_CUDA, "gather_connect: rank %d's buffer: %s", r, cudaGetErrorString(e));
        g->peer[r] = static_cast<float *>(p);
    }
    g->connected = true;
    return FBLT_OK;
}

extern "C" int fblt_gather_rows(fblt_gather *g, const float *rows, size_t nrows, size_t row_offset, void *stream) {
    using namespace fblt;
    NvtxRange nvtx_range("fblt_gather_rows");
    if (!g || (!rows && nrows)) return fail(FBLT_ERR_ARG, "gather_rows: bad arguments");
    if (!g->connected && g->world > 1) return fail(FBLT_ERR_ARG, "gather_rows: fblt_gather_connect has not run");
    if (row_offset + nrows > g->max_rows) return fail(FBLT_ERR_CAPACITY, "gather_rows: %zu rows at %zu exceed the slot of %zu", nrows, row_offset, g->max_rows);
    if (nrows == 0) return FBLT_OK;
    const size_t bytes = nrows * g->row_elems * sizeof(float);
    const size_t slot = ((size_t)g->rank * g->max_rows + row_offset) * g->row_elems;
    for (int i = 0; i < g->world; ++i) {
        const int r = (g->rank + i) % g->world; // every rank starts with its own buffer and walks on from there
        FBLT_CUDA_TRY(cudaMemcpyAsync(g->peer[r] + slot, rows, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    }
    return FBLT_OK;
}

extern "C" float *fblt_gather_buffer(fblt_gather *g) { return g ? g->local : nullptr; }

extern "C" void fblt_gather_destroy(fblt_gather *g) {
    if (!g) return;
    for (int r = 0; r < g->world; ++r)
        if (r != g->rank && g->peer[r]) cudaIpcCloseMemHandle(g->peer[r]);
    if (g->local) cudaFree(g->local);
    delete g;
}
