// Whole forward path behind one C entry point (stages 1-6 sequenced on the caller's stream).
#include <atomic>
#include <chrono>

#include <sched.h>

#include "tg_radix.cuh"

namespace {

constexpr uint32_t kNotArrived = 0xffffffffu;

inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

// Carves the caller's workspace; the same function sizes it.
struct ForwardWorkspace {
    uint32_t* tri_offsets;
    uint64_t* entries;
    // Everything from `status` up to `clear_end` must be zero when the kernels start: one memset.
    uint32_t* status;
    void* scan_scratch;        // binning kernel: finished-CTA counter, totals of its CTAs
    void* tile_scan_scratch;   // device-wide scan of the tile counts (only beyond kTileScanByLastCta tiles)
    uint32_t* long_list;       // work lists of the per-tile sort; only their six head words need clearing
    uint32_t* tile_cursor;     // [tiles]
    uint32_t* tile_order;      // [tiles] launch order of the compositing kernel, when the binning kernel wrote one
    char* clear_end;
    size_t total;

    ForwardWorkspace(void* base, int T, int tiles, uint32_t cap) {
        size_t off = 0;
        auto take = [&](size_t bytes) {
            void* p = base ? (void*)((char*)base + off) : nullptr;
            off += align_up(bytes ? bytes : 1);
            return p;
        };
        tri_offsets = (uint32_t*)take(sizeof(uint32_t) * ((size_t)T + 2));   // [T] = K, [T+1] = longest tile list
        entries = (uint64_t*)take(sizeof(uint64_t) * (size_t)cap);
        status = (uint32_t*)take(sizeof(uint32_t) * 4);
        scan_scratch = take(tg_host::preprocess_scan_scratch_bytes(T));
        tile_scan_scratch = take(tiles > tg::kTileScanByLastCta ? tg_scan_scratch_bytes(tiles) : 0);
        tile_cursor = (uint32_t*)take(sizeof(uint32_t) * (size_t)tiles);
        long_list = (uint32_t*)take(tg_host::tile_sort_scratch_bytes(tiles));
        clear_end = (char*)long_list + 6 * sizeof(uint32_t);
        tile_order = (uint32_t*)take(sizeof(uint32_t) * (size_t)tiles);
        total = off;
    }
};

// One reusable event per (thread, device): marks "K has reached the host".
int scratch_event(cudaEvent_t* out) {
    constexpr int kMaxDevices = 64;
    static thread_local cudaEvent_t events[kMaxDevices] = {};
    int dev = 0;
    TG_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) {
        tg_host::set_error("device index %d outside the supported range", dev);
        return TG_ERR_BAD_ARG;
    }
    if (events[dev] == nullptr) TG_CUDA(cudaEventCreateWithFlags(&events[dev], cudaEventDisableTiming));
    *out = events[dev];
    return TG_OK;
}

struct StageTimer {
    cudaEvent_t ev[6];
    int n = 0;
    bool on;
    cudaStream_t s;
    StageTimer(bool enable, cudaStream_t stream) : on(enable), s(stream) {
        if (on) for (auto& e : ev) cudaEventCreate(&e);
    }
    void mark() { if (on && n < 6) cudaEventRecord(ev[n++], s); }
    ~StageTimer() { if (on) for (auto& e : ev) cudaEventDestroy(e); }
};

}  // namespace

// Everything before compositing: per-triangle records, tile offsets, sorted tile lists (timer marks 0-3).
static int build_tile_lists(const float* vertices, const int32_t* indices, const float* colors, const float* opacities,
                            int T, int W, int H, int tw, int th, int max_layers, float* tri_geo, float* tri_attr,
                            int32_t* sorted_ids, uint32_t list_capacity, int32_t* offsets, void* workspace,
                            size_t workspace_bytes, uint32_t* info_host, unsigned flags, StageTimer& timer,
                            uint32_t** device_status, const uint32_t** tile_order_out, cudaStream_t s) {
    TG_REQUIRE(T >= 0 && W > 0 && H > 0 && tw > 0 && th > 0, "sizes");
    TG_REQUIRE(tw * th <= 1024, "tile_width * tile_height must be <= 1024");
    TG_REQUIRE(max_layers >= 1, "max_layers must be >= 1");
    TG_REQUIRE(workspace && info_host && offsets, "null pointer");
    TG_REQUIRE(((uintptr_t)workspace & 255) == 0, "workspace must be 256-byte aligned");
    TG_REQUIRE(list_capacity < 0x80000000u, "list capacity must stay below 2^31");
    const int tiles_x = (W + tw - 1) / tw, tiles_y = (H + th - 1) / th;
    const int tiles = tiles_x * tiles_y;
    TG_REQUIRE((flags & ~(unsigned)(TG_FORWARD_CULL_TILES | TG_INPUT_PACKED)) == 0, "unknown flag");
    const bool packed = (flags & TG_INPUT_PACKED) != 0;
    // beyond 65536 tiles the tile counts go through the device-wide scan, which the culling variant does not feed
    const bool cull = (flags & TG_FORWARD_CULL_TILES) != 0 && tiles <= tg::kTileScanByLastCta;
    const ForwardWorkspace ws(workspace, T, tiles, list_capacity);
    *device_status = ws.status;
    *tile_order_out = nullptr;
    if (workspace_bytes < ws.total) {
        tg_host::set_error("forward workspace: need %zu bytes, got %zu", ws.total, workspace_bytes);
        return TG_ERR_WORKSPACE;
    }
    info_host[0] = kNotArrived;     // K < 2^31, so this value means "the copy of K has not landed yet"
    info_host[1] = 0;
    info_host[2] = 0;
    TG_REQUIRE(list_capacity == 0 || sorted_ids != nullptr, "null sorted_ids");
    cudaEvent_t k_ready;
    if (int st = scratch_event(&k_ready)) return st;

    timer.mark();                                                    // [0] start of "init"
    // error word, scan tickets and look-back words, tile counters, head of the sort's work list: one clear
    TG_CUDA(cudaMemsetAsync(ws.status, 0, (size_t)(ws.clear_end - (char*)ws.status), s));
    timer.mark();                                                    // [1] start of "bary_transforms"
    // per-triangle records, triangle offsets, per-tile counts and tile offsets
    int st = tg_host::preprocess_scan(vertices, indices, colors, opacities, T, W, H, tw, th, tri_geo, tri_attr,
                                      ws.tri_offsets, ws.scan_scratch, ws.status, ws.tile_cursor, offsets,
                                      ws.tile_scan_scratch, cull, packed, ws.tile_order, s);
    if (st) return st;
    timer.mark();                                                    // [2] start of "per_tile_lists"
    TG_CUDA(cudaMemcpyAsync(&info_host[0], ws.tri_offsets + T, 2 * sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
    TG_CUDA(cudaEventRecord(k_ready, s));
    // Entries are written while K travels to the host: the kernel drops those beyond the capacity, and
    // nothing that reads them is launched before K has been checked.
    st = tg_host::emit_entries(vertices, indices, T, W, H, tw, th, ws.tri_offsets, ws.scan_scratch, ws.tile_cursor,
                               ws.entries, list_capacity, cull ? tri_geo : nullptr, packed, s);
    if (st) return st;
    // K arrives by an 8-byte copy into (preferably pinned) host memory.  Watching the word itself is quicker than
    // waking up from cudaEventSynchronize (the compositing kernels cannot be launched before K is known, so every
    // microsecond here is an idle GPU once the entry writer has finished); after a bounded while, or for pageable
    // memory where the copy has completed by now anyway, the event is waited for in the ordinary way, which also
    // surfaces any error of the kernels before it.
    {
        const volatile uint32_t* watched = info_host;
        const auto t0 = std::chrono::steady_clock::now();
        for (uint32_t spins = 1; *watched == kNotArrived; ++spins) {
#if defined(__x86_64__)
            __builtin_ia32_pause();
#endif
            // after a short pure spin the core is offered to other runnable threads between looks (several ranks or
            // issuing threads per core: a waiter must not hold up the thread whose launches it is waiting behind)
            if (spins > 2048) sched_yield();
            if ((spins & 0xfffu) == 0 && std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(200)) break;
        }
        std::atomic_thread_fence(std::memory_order_acquire);
        if (info_host[0] == kNotArrived) TG_CUDA(cudaEventSynchronize(k_ready));
    }
    if (info_host[0] == kNotArrived) {
        tg_host::set_error("the number of list entries never reached the host");
        return TG_ERR_CUDA;
    }
    const uint32_t K = info_host[0];
    // the longest-list word carries "a launch order of the tiles was written" in its top bit
    const bool have_order = (info_host[1] & tg::kOrderWrittenBit) != 0 && info_host[1] != UINT32_MAX;
    if (info_host[1] != UINT32_MAX) info_host[1] &= ~tg::kOrderWrittenBit;
    *tile_order_out = have_order ? ws.tile_order : nullptr;
    if (K > list_capacity) {
        tg_host::set_error("K = %u exceeds the list capacity %u", K, list_capacity);
        return TG_ERR_CAPACITY;
    }
    timer.mark();                                                    // [3] start of "sorting"
    if (K > 0) {
        st = tg_host::sort_tile_lists(ws.entries, offsets, tiles, sorted_ids, ws.long_list, true, false, info_host[1], s);
        if (st) return st;
    }
    return TG_OK;
}

// Stage times from the timer's six marks (synchronises), then the device error word.
static int finish_timing(StageTimer& timer, float* stage_ms_host, const uint32_t* info_host, cudaStream_t s) {
    if (!stage_ms_host) return TG_OK;
    TG_CUDA(cudaStreamSynchronize(s));
    float ms[5];
    for (int i = 0; i < 5; i++) TG_CUDA(cudaEventElapsedTime(&ms[i], timer.ev[i], timer.ev[i + 1]));
    stage_ms_host[0] = ms[0];   // init
    stage_ms_host[1] = ms[2];   // per_tile_lists: K read-back + entry emission
    stage_ms_host[2] = ms[3];   // sorting: per-tile sort
    stage_ms_host[3] = ms[1];   // bary_transforms: preprocess + scan + tile counts and offsets
    stage_ms_host[4] = ms[4];   // rasterization
    if (info_host[2]) {
        tg_host::set_error("device error word = %u", info_host[2]);
        return TG_ERR_DEVICE_FLAG;
    }
    return TG_OK;
}

extern "C" {

size_t tg_forward_workspace_bytes(int T, int tiles, uint32_t list_capacity) {
    if (T < 0) T = 0;
    if (tiles < 0) tiles = 0;
    return ForwardWorkspace(nullptr, T, tiles, list_capacity).total;
}

int tg_render_forward(const float* vertices, const int32_t* indices, const float* colors, const float* opacities, int T,
                      int W, int H, int tw, int th, float thr, int per_pixel_sort, int max_layers, float* image,
                      float* depthmap, float* final_weights, int32_t* ends, int32_t* selection, float* tri_geo,
                      float* tri_attr, int32_t* sorted_ids, uint32_t list_capacity, int32_t* offsets, void* workspace,
                      size_t workspace_bytes, uint32_t* info_host, float* stage_ms_host, unsigned flags,
                      tg_stream_t stream) {
    TG_REQUIRE(image && depthmap && final_weights && ends, "null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    StageTimer timer(stage_ms_host != nullptr, s);
    uint32_t* device_status = nullptr;
    const uint32_t* tile_order = nullptr;
    int st = build_tile_lists(vertices, indices, colors, opacities, T, W, H, tw, th, max_layers, tri_geo, tri_attr,
                              sorted_ids, list_capacity, offsets, workspace, workspace_bytes, info_host, flags, timer, &device_status, &tile_order, s);
    if (st) return st;
    timer.mark();                                                    // [4] start of "rasterization"
    tg_host::set_tile_order(tile_order, info_host[1]);      // with the longest list: long lists are streamed
    st = tg_blend_forward(tri_geo, tri_attr, sorted_ids, offsets, W, H, tw, th, thr, per_pixel_sort, max_layers, image,
                          depthmap, final_weights, ends, selection, stream);
    tg_host::set_tile_order(nullptr);
    if (st) return st;
    timer.mark();                                                    // [5] end
    // device error word: valid on the host once the stream has been synchronised
    TG_CUDA(cudaMemcpyAsync(&info_host[2], device_status, sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
    return finish_timing(timer, stage_ms_host, info_host, s);
}

int tg_render_step_l2(const float* vertices, const int32_t* indices, const float* colors, const float* opacities, int T,
                      int V, int W, int H, int tw, int th, float thr, int max_layers, const float* target,
                      float grad_scale, float loss_scale, float* loss_out, float* image, float* depthmap,
                      float* final_weights, int32_t* ends, float* tri_geo, float* tri_attr, int32_t* sorted_ids,
                      uint32_t list_capacity, int32_t* offsets, float* grad_vertices, float* grad_colors,
                      float* grad_opacities, int accumulate, void* workspace, size_t workspace_bytes, void* scratch,
                      size_t scratch_bytes, uint32_t* info_host, float* stage_ms_host, unsigned flags,
                      tg_stream_t stream) {
    TG_REQUIRE(image && depthmap && final_weights && ends && target, "null pointer");
    TG_REQUIRE(tw * th <= 256 && max_layers <= 32, "the one-kernel step needs tiles of at most 256 pixels and max_layers <= 32");
    cudaStream_t s = (cudaStream_t)stream;
    StageTimer timer(stage_ms_host != nullptr, s);
    uint32_t* device_status = nullptr;
    const uint32_t* tile_order = nullptr;
    int st = build_tile_lists(vertices, indices, colors, opacities, T, W, H, tw, th, max_layers, tri_geo, tri_attr,
                              sorted_ids, list_capacity, offsets, workspace, workspace_bytes, info_host, flags, timer, &device_status, &tile_order, s);
    if (st) return st;
    timer.mark();                                                    // [4] start of "rasterization" (here: forward + backward)
    tg_host::set_tile_order(tile_order);
    st = tg_blend_step_l2(tri_geo, tri_attr, sorted_ids, offsets, V, W, H, tw, th, thr, max_layers, target, grad_scale,
                          loss_scale, loss_out, image, depthmap, final_weights, ends, grad_vertices, grad_colors,
                          grad_opacities, accumulate, scratch, scratch_bytes, stream);
    tg_host::set_tile_order(nullptr);
    if (st) return st;
    timer.mark();                                                    // [5] end
    TG_CUDA(cudaMemcpyAsync(&info_host[2], device_status, sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
    return finish_timing(timer, stage_ms_host, info_host, s);
}

}  // extern "C"
