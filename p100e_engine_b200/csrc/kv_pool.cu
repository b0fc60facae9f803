// Paged KV pool, block tables, step descriptors, page offload and the sequence file format: the caller-side structures
// the attention kernels index, as host C++ behind the C ABI.
//
// Reference counterparts (src/tp_model.cu in the reference project): alloc_pool :3880-3966 (one allocation per GPU laid out
// [K|V][kv layer][page][2^psh positions][row]), ensure_pages :3358-3384 (free list, stream-ordered upload of new table
// entries from a pinned row), forward_batch_ids :3999-4022 (per-row positions and table offsets rtab[row] = slot *
// max_pages), kv_seq / kv_rows :3327-3337 (the cache views handed to the kernels), seq_offload / pages_out :3432-3481,
// :3676-3686 (host layout [page][K|V][kv layer][page rows], two 2-D copies per page) and seq_write / seq_read :3738-3862
// (magic "P100ESQ2", 15 x u64 fingerprint, n_past / n_tok / pages, tokens, then per GPU its pages and state).
// Differences: all offsets are 64-bit (a layer region may exceed 4 GiB), a step may hold any number of rows, and a pool
// may be one of n_seq sequence shards: the pages of a sequence are dealt round-robin over the shards (logical page g lives
// on shard g mod n_seq as that shard's local page g / n_seq), so positions given to this API are global and the pool
// converts them.  A pool can also live in host memory (device < 0): the same code paths with memcpy, for tools and tests.
#include "common.cuh"

#include <algorithm>
#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <unistd.h>
#include <vector>

struct b200_pool {
    uint32_t type;
    int Hkv, D, n_layers, n_pages, psh, max_slots, max_pages, n_seq, seq_rank, dev;
    size_t rowb, pblk, region, total;
    char * base;
    int32_t * ptab_h, * ptab_d;
    std::vector<int32_t> free_pages;
    std::vector<int32_t> n_alloc;
    // step descriptor: [pos_g | pos_l | crow | rtab] x max_rows, two pinned staging buffers used in turn
    int max_rows, rows, max_n, turn;
    void * step_stream = nullptr;   // the stream of the last step (whose attention calls share one split plan)
    bool stepped = false;
    int32_t * step_h[2], * step_d;
    cudaEvent_t step_ev[2];
    bool ev_used[2];
};

namespace {

using namespace b200;

bool on_device(const b200_pool * p) { return p->dev >= 0; }

uint64_t splitmix(uint64_t & s) {
    uint64_t z = (s += 0x9e3779b97f4a7c15ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

// global position -> local position of the last key of this shard that a row at `pos` sees (-1: none), and whether the
// shard owns `pos` itself
int local_last(const b200_pool * p, long long pos, bool * owns) {
    if (owns) *owns = false;
    if (pos < 0) return -1;
    const long long ps = 1ll << p->psh, g = pos >> p->psh, o = pos & (ps - 1);
    long long before = (g - p->seq_rank + p->n_seq - 1) / p->n_seq;   // owned pages with index < g
    if (before < 0) before = 0;
    const bool own = g % p->n_seq == p->seq_rank;
    if (owns) *owns = own;
    return (int) (own ? before * ps + o : before * ps - 1);
}
int local_len(const b200_pool * p, long long n) { return n <= 0 ? 0 : local_last(p, n - 1, nullptr) + 1; }

int copy_rows(const b200_pool * p, void * dst, size_t dpitch, const void * src, size_t spitch, size_t width, size_t height,
              bool to_host, cudaStream_t s) {
    if (!on_device(p)) {
        for (size_t i = 0; i < height; ++i) memcpy((char *) dst + i * dpitch, (const char *) src + i * spitch, width);
        return B200_OK;
    }
    const cudaError_t e = cudaMemcpy2DAsync(dst, dpitch, src, spitch, width, height, to_host ? cudaMemcpyDeviceToHost : cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) { cudaGetLastError(); fprintf(stderr, "b200attn: pool page copy: %s\n", cudaGetErrorString(e)); return B200_ERR_CUDA; }
    return B200_OK;
}

int write_all(int fd, const void * buf, size_t n) {
    const char * p = (const char *) buf;
    while (n) {
        const ssize_t w = write(fd, p, n);
        if (w < 0) { if (errno == EINTR) continue; return B200_ERR_IO; }
        p += w; n -= (size_t) w;
    }
    return B200_OK;
}
int read_all(int fd, void * buf, size_t n) {
    char * p = (char *) buf;
    while (n) {
        const ssize_t r = read(fd, p, n);
        if (r < 0) { if (errno == EINTR) continue; return B200_ERR_IO; }
        if (r == 0) return B200_ERR_FORMAT;   // short file
        p += r; n -= (size_t) r;
    }
    return B200_OK;
}

const char SEQ_MAGIC[8] = {'P', '1', '0', '0', 'E', 'S', 'Q', '2'};

}  // namespace

extern "C" {

void b200_pool_destroy(b200_pool * p);

b200_pool * b200_pool_create(uint32_t kv_type, int Hkv, int D, int n_layers, int n_pages, int psh, int max_slots, int max_pages,
                             int max_rows, uint32_t seed, int n_seq, int seq_rank, int device) {
    if ((kv_type != B200_KV_F16 && kv_type != B200_KV_Q8_0 && kv_type != B200_KV_Q4_0) || Hkv < 1 || D < 32 || D % 32 || n_layers < 1 ||
        n_pages < 1 || psh < 0 || psh > 20 || max_slots < 1 || max_pages < 1 || max_rows < 1 || n_seq < 1 || seq_rank < 0 || seq_rank >= n_seq) {
        fprintf(stderr, "b200attn: pool_create: unsupported arguments\n");
        return nullptr;
    }
    b200_pool * p = new b200_pool();
    p->type = kv_type; p->Hkv = Hkv; p->D = D; p->n_layers = n_layers; p->n_pages = n_pages; p->psh = psh;
    p->max_slots = max_slots; p->max_pages = max_pages; p->n_seq = n_seq; p->seq_rank = seq_rank; p->dev = device;
    p->rowb = (size_t) Hkv * head_bytes(kv_type, D);
    p->pblk = p->rowb << psh;
    p->region = (size_t) n_pages * p->pblk;
    p->total = 2 * (size_t) n_layers * p->region;
    p->max_rows = max_rows; p->rows = 0; p->max_n = 0; p->turn = 0;
    p->ev_used[0] = p->ev_used[1] = false;
    const size_t tab_bytes = (size_t) max_slots * max_pages * sizeof(int32_t), step_bytes = (size_t) 4 * max_rows * sizeof(int32_t);
    bool ok = true;
    if (device >= 0) {
        ok = cudaSetDevice(device) == cudaSuccess && cudaMalloc(&p->base, p->total) == cudaSuccess &&
             cudaMemset(p->base, 0, p->total) == cudaSuccess &&   // unused tail rows of a page read as zeros (finite, weight 0)
             cudaMalloc(&p->ptab_d, tab_bytes) == cudaSuccess && cudaHostAlloc(&p->ptab_h, tab_bytes, cudaHostAllocPortable) == cudaSuccess &&
             cudaMalloc(&p->step_d, step_bytes) == cudaSuccess && cudaHostAlloc(&p->step_h[0], step_bytes, cudaHostAllocPortable) == cudaSuccess &&
             cudaHostAlloc(&p->step_h[1], step_bytes, cudaHostAllocPortable) == cudaSuccess &&
             cudaEventCreateWithFlags(&p->step_ev[0], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&p->step_ev[1], cudaEventDisableTiming) == cudaSuccess;
    } else {
        p->base = (char *) calloc(p->total, 1);
        p->ptab_h = (int32_t *) malloc(tab_bytes);
        p->ptab_d = p->ptab_h;
        p->step_h[0] = (int32_t *) malloc(step_bytes);
        p->step_h[1] = p->step_h[0];
        p->step_d = p->step_h[0];
        ok = p->base && p->ptab_h && p->step_h[0];
    }
    if (!ok) {
        if (device >= 0) cudaGetLastError();
        fprintf(stderr, "b200attn: pool_create: allocation of %zu bytes failed\n", p->total);
        b200_pool_destroy(p);   // releases whatever was allocated
        return nullptr;
    }
    for (size_t i = 0; i < (size_t) max_slots * max_pages; ++i) p->ptab_h[i] = -1;
    if (device >= 0) cudaMemcpy(p->ptab_d, p->ptab_h, tab_bytes, cudaMemcpyHostToDevice);
    // pages are handed out from the back of the list: ascending ids, or a seeded shuffle (a long-running server's scatter)
    p->free_pages.resize(n_pages);
    for (int i = 0; i < n_pages; ++i) p->free_pages[i] = n_pages - 1 - i;
    if (seed) {
        uint64_t s = seed;
        for (int i = n_pages - 1; i > 0; --i) std::swap(p->free_pages[i], p->free_pages[(size_t) (splitmix(s) % (uint64_t) (i + 1))]);
    }
    p->n_alloc.assign(max_slots, 0);
    return p;
}

void b200_pool_destroy(b200_pool * p) {
    if (!p) return;
    if (on_device(p)) {
        cudaSetDevice(p->dev);
        if (p->stepped) b200_attn_step_end(p->step_stream);   // its step descriptor is about to go away
        if (p->base) cudaFree(p->base);
        if (p->ptab_d) cudaFree(p->ptab_d);
        if (p->ptab_h) cudaFreeHost(p->ptab_h);
        if (p->step_d) cudaFree(p->step_d);
        for (int i = 0; i < 2; ++i) {
            if (p->step_h[i]) cudaFreeHost(p->step_h[i]);
            if (p->step_ev[i]) cudaEventDestroy(p->step_ev[i]);
        }
        cudaGetLastError();
    } else {
        free(p->base);
        free(p->ptab_h);
        free(p->step_h[0]);
    }
    delete p;
}

size_t b200_pool_bytes(const b200_pool * p) { return p ? p->total : 0; }
size_t b200_pool_page_bytes(const b200_pool * p) { return p ? 2 * (size_t) p->n_layers * p->pblk : 0; }
int b200_pool_free_pages(const b200_pool * p) { return p ? (int) p->free_pages.size() : 0; }
int b200_pool_slot_pages(const b200_pool * p, int slot) { return p && slot >= 0 && slot < p->max_slots ? p->n_alloc[slot] : -1; }
const int32_t * b200_pool_table_host(const b200_pool * p) { return p ? p->ptab_h : nullptr; }
void * b200_pool_base(const b200_pool * p) { return p ? p->base : nullptr; }
int b200_pool_local_length(const b200_pool * p, int n_positions) { return p ? local_len(p, n_positions) : 0; }

// raw bytes of the pool -> dst (host or device memory), asynchronous on the stream; for tools that inspect or checkpoint pages
int b200_pool_read(const b200_pool * p, size_t offset, void * dst, size_t nbytes, void * stream) {
    if (!p || !dst || offset > p->total || nbytes > p->total - offset) B200_REFUSE(B200_ERR_SHAPE, "pool_read: range outside the pool");
    if (!on_device(p)) { memcpy(dst, p->base + offset, nbytes); return B200_OK; }
    const cudaError_t e = cudaMemcpyAsync(dst, p->base + offset, nbytes, cudaMemcpyDefault, (cudaStream_t) stream);
    if (e != cudaSuccess) { cudaGetLastError(); B200_REFUSE(B200_ERR_CUDA, "pool_read: %s", cudaGetErrorString(e)); }
    return B200_OK;
}

// ensure_pages: make global positions [0, n_positions) of the slot addressable on this shard.  New table entries go to the
// device with one stream-ordered copy from the pinned row (entries already uploaded are never rewritten while in flight).
int b200_pool_ensure(b200_pool * p, int slot, int n_positions, void * stream) {
    if (!p || slot < 0 || slot >= p->max_slots || n_positions < 0) B200_REFUSE(B200_ERR_SHAPE, "pool_ensure: bad slot / length");
    const int n_loc = local_len(p, n_positions);
    const int need = (int) (((long long) n_loc + (1ll << p->psh) - 1) >> p->psh), have = p->n_alloc[slot];
    if (need <= have) return B200_OK;
    if (need > p->max_pages) B200_REFUSE(B200_ERR_SHAPE, "pool_ensure: context full (%d pages needed, %d per sequence)", need, p->max_pages);
    if (need - have > (int) p->free_pages.size())
        B200_REFUSE(B200_ERR_ALLOC, "pool_ensure: KV pool full (%zu free pages, need %d)", p->free_pages.size(), need - have);
    int32_t * row = p->ptab_h + (size_t) slot * p->max_pages;
    for (int i = have; i < need; ++i) { row[i] = p->free_pages.back(); p->free_pages.pop_back(); }
    p->n_alloc[slot] = need;
    if (on_device(p)) {
        const cudaError_t e = cudaMemcpyAsync(p->ptab_d + (size_t) slot * p->max_pages + have, row + have, (size_t) (need - have) * sizeof(int32_t),
                                              cudaMemcpyHostToDevice, (cudaStream_t) stream);
        if (e != cudaSuccess) { cudaGetLastError(); B200_REFUSE(B200_ERR_CUDA, "pool_ensure: table upload: %s", cudaGetErrorString(e)); }
    }
    return B200_OK;
}

// give the slot's pages back (the caller has made sure no kernel still reads them, as the reference does through sync_all)
int b200_pool_release(b200_pool * p, int slot, void * stream) {
    if (!p || slot < 0 || slot >= p->max_slots) B200_REFUSE(B200_ERR_SHAPE, "pool_release: bad slot");
    int32_t * row = p->ptab_h + (size_t) slot * p->max_pages;
    for (int i = p->n_alloc[slot] - 1; i >= 0; --i) { p->free_pages.push_back(row[i]); row[i] = -1; }
    const int had = p->n_alloc[slot];
    p->n_alloc[slot] = 0;
    if (on_device(p) && had) {
        // the pinned row now holds -1 in the released entries; the upload is stream-ordered after the slot's last use
        const cudaError_t e = cudaMemcpyAsync(p->ptab_d + (size_t) slot * p->max_pages, row, (size_t) had * sizeof(int32_t), cudaMemcpyHostToDevice,
                                              (cudaStream_t) stream);
        if (e != cudaSuccess) { cudaGetLastError(); B200_REFUSE(B200_ERR_CUDA, "pool_release: table upload: %s", cudaGetErrorString(e)); }
    }
    return B200_OK;
}

// kv_seq (slot >= 0: that sequence's table, no per-row offsets) / kv_rows (slot < 0: the whole table with the step's rtab)
int b200_pool_view(const b200_pool * p, int layer, int slot, b200_kv_cache * out) {
    if (!p || !out || layer < 0 || layer >= p->n_layers || slot >= p->max_slots) B200_REFUSE(B200_ERR_SHAPE, "pool_view: bad layer / slot");
    out->type = p->type; out->n_ctx = p->max_pages << p->psh; out->Hkv = p->Hkv; out->D = p->D;
    out->k = p->base + (size_t) layer * p->region;
    out->v = p->base + (size_t) (p->n_layers + layer) * p->region;
    out->psh = p->psh; out->pstride = p->pblk;
    if (slot >= 0) { out->pt = p->ptab_d + (size_t) slot * p->max_pages; out->rtab = nullptr; }
    else { out->pt = p->ptab_d; out->rtab = p->step_d + 3 * (size_t) p->max_rows; }
    return B200_OK;
}

// Step descriptor of a decode / verify step: row r = i * q_len + j is token j of slots[i] at global position
// n_past[i] + j (host arrays).  Uploads, stream-ordered from pinned memory, per row: the global (rotary) position, the local
// position of the last key this shard holds for the row (-1: none), the local cache row where the row's own K/V goes (-1: the
// page belongs to another shard) and rtab[r] = slot * max_pages.  grow != 0 also makes the new positions addressable.
int b200_pool_step(b200_pool * p, const int32_t * slots, const int32_t * n_past, int n, int q_len, int grow, void * stream) {
    if (!p || !slots || !n_past || n < 1 || q_len < 1 || (long long) n * q_len > p->max_rows) B200_REFUSE(B200_ERR_SHAPE, "pool_step: bad batch (rows %lld, capacity %d)", (long long) n * q_len, p ? p->max_rows : 0);
    for (int i = 0; i < n; ++i)
        if (slots[i] < 0 || slots[i] >= p->max_slots || n_past[i] < 0) B200_REFUSE(B200_ERR_SHAPE, "pool_step: bad slot / position at %d", i);
    if (grow)
        for (int i = 0; i < n; ++i) {
            const int rc = b200_pool_ensure(p, slots[i], n_past[i] + q_len, stream);
            if (rc != B200_OK) return rc;
        }
    const int turn = p->turn;
    cudaStream_t s = (cudaStream_t) stream;
    if (on_device(p) && p->ev_used[turn]) cudaEventSynchronize(p->step_ev[turn]);   // this staging buffer's last upload has left
    int32_t * h = p->step_h[turn];
    const int mr = p->max_rows;
    int max_n = 0;
    for (int i = 0; i < n; ++i)
        for (int j = 0; j < q_len; ++j) {
            const int r = i * q_len + j, pos = n_past[i] + j;
            bool own;
            const int loc = local_last(p, pos, &own);
            h[r] = pos; h[mr + r] = loc; h[2 * mr + r] = own ? loc : -1; h[3 * mr + r] = slots[i] * p->max_pages;
            max_n = std::max(max_n, loc + 1);
        }
    p->rows = n * q_len;
    p->max_n = std::max(max_n, 1);
    if (on_device(p)) {
        for (int part = 0; part < 4; ++part) {
            const cudaError_t e = cudaMemcpyAsync(p->step_d + (size_t) part * mr, h + (size_t) part * mr, (size_t) p->rows * sizeof(int32_t),
                                                  cudaMemcpyHostToDevice, s);
            if (e != cudaSuccess) { cudaGetLastError(); B200_REFUSE(B200_ERR_CUDA, "pool_step: upload: %s", cudaGetErrorString(e)); }
        }
        cudaEventRecord(p->step_ev[turn], s);
        p->ev_used[turn] = true;
        p->turn ^= 1;
        // the positions of this step are now fixed: the batched attention calls on this stream may share one split plan
        const int rc = b200_attn_step_begin(stream, p->step_d, 4 * (size_t) mr * sizeof(int32_t));
        if (rc != B200_OK) return rc;
        p->step_stream = stream;
        p->stepped = true;
    }
    return B200_OK;
}
const int32_t * b200_pool_step_rope_pos(const b200_pool * p) { return p ? p->step_d : nullptr; }
const int32_t * b200_pool_step_last_key(const b200_pool * p) { return p ? p->step_d + (size_t) p->max_rows : nullptr; }
const int32_t * b200_pool_step_cache_row(const b200_pool * p) { return p ? p->step_d + 2 * (size_t) p->max_rows : nullptr; }
const int32_t * b200_pool_step_rtab(const b200_pool * p) { return p ? p->step_d + 3 * (size_t) p->max_rows : nullptr; }
int b200_pool_step_rows(const b200_pool * p) { return p ? p->rows : 0; }
int b200_pool_step_max_n(const b200_pool * p) { return p ? p->max_n : 0; }

// pages first .. first+n-1 of the slot -> dst in the offload layout [page][K|V][layer][page rows] (page_bytes each):
// two 2-D copies per page (K blocks of all layers, V blocks of all layers), asynchronous on the stream
int b200_pool_pages_out(const b200_pool * p, int slot, int first, int n, void * dst, void * stream) {
    if (!p || !dst || slot < 0 || slot >= p->max_slots || first < 0 || n < 0 || first + n > p->n_alloc[slot]) B200_REFUSE(B200_ERR_SHAPE, "pool_pages_out: bad page range");
    const size_t pb = 2 * (size_t) p->n_layers * p->pblk;
    const int32_t * row = p->ptab_h + (size_t) slot * p->max_pages;
    for (int i = 0; i < n; ++i)
        for (int kv = 0; kv < 2; ++kv) {
            const int rc = copy_rows(p, (char *) dst + (size_t) i * pb + (size_t) kv * p->n_layers * p->pblk, p->pblk,
                                     p->base + (size_t) kv * p->n_layers * p->region + (size_t) row[first + i] * p->pblk, p->region, p->pblk,
                                     (size_t) p->n_layers, true, (cudaStream_t) stream);
            if (rc != B200_OK) return rc;
        }
    return B200_OK;
}
// the reverse: the slot receives pages first .. first+n-1 from src (pages are taken from the free list as needed)
int b200_pool_pages_in(b200_pool * p, int slot, int first, int n, const void * src, void * stream) {
    if (!p || !src || slot < 0 || slot >= p->max_slots || first < 0 || n < 0 || first > p->n_alloc[slot]) B200_REFUSE(B200_ERR_SHAPE, "pool_pages_in: bad page range");
    if (first + n > p->max_pages) B200_REFUSE(B200_ERR_SHAPE, "pool_pages_in: more pages than a sequence may hold");
    const int extra = first + n - p->n_alloc[slot];
    if (extra > (int) p->free_pages.size()) B200_REFUSE(B200_ERR_ALLOC, "pool_pages_in: KV pool full");
    int32_t * row = p->ptab_h + (size_t) slot * p->max_pages;
    const int have = p->n_alloc[slot];
    for (int i = have; i < first + n; ++i) { row[i] = p->free_pages.back(); p->free_pages.pop_back(); }
    if (extra > 0) {
        p->n_alloc[slot] = first + n;
        if (on_device(p) && cudaMemcpyAsync(p->ptab_d + (size_t) slot * p->max_pages + have, row + have, (size_t) extra * sizeof(int32_t),
                                            cudaMemcpyHostToDevice, (cudaStream_t) stream) != cudaSuccess) {
            cudaGetLastError();
            B200_REFUSE(B200_ERR_CUDA, "pool_pages_in: table upload failed");
        }
    }
    const size_t pb = 2 * (size_t) p->n_layers * p->pblk;
    for (int i = 0; i < n; ++i)
        for (int kv = 0; kv < 2; ++kv) {
            const int rc = copy_rows(p, p->base + (size_t) kv * p->n_layers * p->region + (size_t) row[first + i] * p->pblk, p->region,
                                     (const char *) src + (size_t) i * pb + (size_t) kv * p->n_layers * p->pblk, p->pblk, p->pblk,
                                     (size_t) p->n_layers, false, (cudaStream_t) stream);
            if (rc != B200_OK) return rc;
        }
    return B200_OK;
}

// ---- sequence file ---------------------------------------------------------------------------------------------
// "P100ESQ2" | fingerprint (15 x u64) | n_past, n_tok, pages (i32) | tokens (i32 x n_tok) | per GPU: pages x page_bytes in
// the offload layout, then that GPU's recurrent state (opaque here: the other mixers' state is the caller's).
int b200_session_write_header(int fd, const uint64_t * fingerprint, int n_past, const int32_t * tokens, int n_tok, int pages) {
    if (!fingerprint || n_past < 0 || n_tok < 0 || pages < 0 || (n_tok && !tokens)) B200_REFUSE(B200_ERR_SHAPE, "session_write_header: bad arguments");
    const int32_t hdr[3] = {n_past, n_tok, pages};
    int rc = write_all(fd, SEQ_MAGIC, 8);
    if (rc == B200_OK) rc = write_all(fd, fingerprint, 15 * sizeof(uint64_t));
    if (rc == B200_OK) rc = write_all(fd, hdr, sizeof hdr);
    if (rc == B200_OK) rc = write_all(fd, tokens, (size_t) n_tok * sizeof(int32_t));
    if (rc != B200_OK) fprintf(stderr, "b200attn: session_write_header: write failed (disk full?)\n");
    return rc;
}
// this GPU's block: the slot's pages (through a staging buffer of up to 32 pages; synchronises the stream per batch) + state
int b200_session_write_rank(int fd, const b200_pool * p, int slot, int pages, const void * state, size_t state_bytes, void * stream) {
    if (!p || slot < 0 || slot >= p->max_slots || pages < 0 || pages > p->n_alloc[slot] || (state_bytes && !state)) B200_REFUSE(B200_ERR_SHAPE, "session_write_rank: bad arguments");
    const size_t pb = b200_pool_page_bytes(p);
    const int chunk = std::max(1, std::min(pages, 32));
    char * st = nullptr;
    if (on_device(p)) { if (cudaHostAlloc(&st, (size_t) chunk * pb, cudaHostAllocPortable) != cudaSuccess) { cudaGetLastError(); st = nullptr; } }
    else st = (char *) malloc((size_t) chunk * pb);
    if (!st) B200_REFUSE(B200_ERR_ALLOC, "session_write_rank: staging allocation failed");
    int rc = B200_OK;
    for (int p0 = 0; p0 < pages && rc == B200_OK; p0 += chunk) {
        const int n = std::min(chunk, pages - p0);
        rc = b200_pool_pages_out(p, slot, p0, n, st, stream);
        if (rc == B200_OK && on_device(p) && cudaStreamSynchronize((cudaStream_t) stream) != cudaSuccess) { cudaGetLastError(); rc = B200_ERR_CUDA; }
        if (rc == B200_OK) rc = write_all(fd, st, (size_t) n * pb);
    }
    if (rc == B200_OK) rc = write_all(fd, state, state_bytes);
    if (on_device(p)) cudaFreeHost(st); else free(st);
    if (rc == B200_ERR_IO) fprintf(stderr, "b200attn: session_write_rank: write failed (disk full?)\n");
    return rc;
}
// Reads and checks the header.  *bad_field: -1, or the index of the first fingerprint field that differs from `want`
// (7 = GPU count / split, as in the reference's message).  tokens receives n_tok ids (capacity tok_cap).
int b200_session_read_header(int fd, const uint64_t * want, int max_ctx, int max_pages, int psh, int * n_past, int * n_tok, int * pages,
                             int32_t * tokens, int tok_cap, int * bad_field) {
    if (bad_field) *bad_field = -1;
    if (!want || !n_past || !n_tok || !pages) B200_REFUSE(B200_ERR_SHAPE, "session_read_header: null argument");
    char mg[8];
    int rc = read_all(fd, mg, 8);
    if (rc != B200_OK) B200_REFUSE(rc, "session_read_header: short file");
    if (!memcmp(mg, "P100ESQ1", 8)) B200_REFUSE(B200_ERR_FORMAT, "session_read_header: a version 1 sequence file (no fingerprint): not loadable");
    if (memcmp(mg, SEQ_MAGIC, 8)) B200_REFUSE(B200_ERR_FORMAT, "session_read_header: not a p100e sequence file");
    uint64_t fp[15];
    rc = read_all(fd, fp, sizeof fp);
    if (rc != B200_OK) B200_REFUSE(rc, "session_read_header: short file");
    for (int i = 0; i < 15; ++i)
        if (fp[i] != want[i]) {
            if (bad_field) *bad_field = i;
            B200_REFUSE(B200_ERR_FORMAT, "session_read_header: saved with another model / KV layout (fingerprint field %d: %llu vs %llu)", i,
                        (unsigned long long) fp[i], (unsigned long long) want[i]);
        }
    int32_t hdr[3];
    rc = read_all(fd, hdr, sizeof hdr);
    if (rc != B200_OK) B200_REFUSE(rc, "session_read_header: short file");
    if (hdr[0] < 0 || hdr[0] > max_ctx || hdr[1] != hdr[0] || hdr[2] < 0 || hdr[2] > max_pages || ((long long) hdr[2] << psh) < hdr[0])
        B200_REFUSE(B200_ERR_FORMAT, "session_read_header: bad header (or the sequence exceeds this engine's context)");
    if (hdr[1] > tok_cap || (hdr[1] && !tokens)) B200_REFUSE(B200_ERR_SHAPE, "session_read_header: token buffer too small (%d needed)", hdr[1]);
    rc = read_all(fd, tokens, (size_t) hdr[1] * sizeof(int32_t));
    if (rc != B200_OK) B200_REFUSE(rc, "session_read_header: short file");
    *n_past = hdr[0]; *n_tok = hdr[1]; *pages = hdr[2];
    return B200_OK;
}
int b200_session_read_rank(int fd, b200_pool * p, int slot, int pages, void * state, size_t state_bytes, void * stream) {
    if (!p || slot < 0 || slot >= p->max_slots || pages < 0 || pages > p->max_pages || (state_bytes && !state)) B200_REFUSE(B200_ERR_SHAPE, "session_read_rank: bad arguments");
    if (p->n_alloc[slot] != 0) B200_REFUSE(B200_ERR_SHAPE, "session_read_rank: the slot already holds pages");
    const size_t pb = b200_pool_page_bytes(p);
    const int chunk = std::max(1, std::min(pages, 32));
    char * st = nullptr;
    if (on_device(p)) { if (cudaHostAlloc(&st, (size_t) chunk * pb, cudaHostAllocPortable) != cudaSuccess) { cudaGetLastError(); st = nullptr; } }
    else st = (char *) malloc((size_t) chunk * pb);
    if (!st) B200_REFUSE(B200_ERR_ALLOC, "session_read_rank: staging allocation failed");
    int rc = B200_OK;
    for (int p0 = 0; p0 < pages && rc == B200_OK; p0 += chunk) {
        const int n = std::min(chunk, pages - p0);
        rc = read_all(fd, st, (size_t) n * pb);
        if (rc == B200_OK) rc = b200_pool_pages_in(p, slot, p0, n, st, stream);
        if (rc == B200_OK && on_device(p) && cudaStreamSynchronize((cudaStream_t) stream) != cudaSuccess) { cudaGetLastError(); rc = B200_ERR_CUDA; }
    }
    if (rc == B200_OK) rc = read_all(fd, state, state_bytes);
    if (on_device(p)) cudaFreeHost(st); else free(st);
    if (rc != B200_OK) fprintf(stderr, "b200attn: session_read_rank: failed (status %d)\n", rc);
    return rc;
}

}  // extern "C"
