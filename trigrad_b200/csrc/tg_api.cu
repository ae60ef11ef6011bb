// Whole forward path behind one C entry point (stages 1-6 sequenced on the caller's stream).
#include "tg_radix.cuh"

namespace {

inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

inline int ceil_log2(int x) {
    int b = 0;
    while ((1ll << b) < (long long)x) b++;
    return b;
}

// Carves the caller's workspace; the same function sizes it.
struct ForwardWorkspace {
    uint32_t* tri_offsets;
    uint64_t* keys_a;
    uint64_t* keys_b;
    uint32_t* ids_tmp;
    // status word, scan scratch and sort scratch lie back to back: one memset clears all three
    uint32_t* status;
    void* scan_scratch;
    void* sort_scratch;
    size_t sort_scratch_bytes;
    size_t total;

    ForwardWorkspace(void* base, int T, uint32_t cap) {
        size_t off = 0;
        auto take = [&](size_t bytes) {
            void* p = base ? (void*)((char*)base + off) : nullptr;
            off += align_up(bytes ? bytes : 1);
            return p;
        };
        tri_offsets = (uint32_t*)take(sizeof(uint32_t) * ((size_t)T + 1));
        keys_a = (uint64_t*)take(sizeof(uint64_t) * (size_t)cap);
        keys_b = (uint64_t*)take(sizeof(uint64_t) * (size_t)cap);
        ids_tmp = (uint32_t*)take(sizeof(uint32_t) * (size_t)cap);
        status = (uint32_t*)take(sizeof(uint32_t) * 4);
        scan_scratch = take(tg_host::preprocess_scan_scratch_bytes(T));
        sort_scratch_bytes = tg_sort_scratch_bytes(cap);
        sort_scratch = take(sort_scratch_bytes);
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

extern "C" {

size_t tg_forward_workspace_bytes(int T, int tiles, uint32_t list_capacity) {
    (void)tiles;
    if (T < 0) T = 0;
    return ForwardWorkspace(nullptr, T, list_capacity).total;
}

int tg_render_forward(const float* vertices, const int32_t* indices, const float* colors, const float* opacities, int T,
                      int W, int H, int tw, int th, float thr, int per_pixel_sort, int max_layers, float* image,
                      float* depthmap, float* final_weights, int32_t* ends, int32_t* selection, float* tri_geo,
                      float* tri_attr, int32_t* sorted_ids, uint32_t list_capacity, int32_t* offsets, void* workspace,
                      size_t workspace_bytes, uint32_t* info_host, float* stage_ms_host, tg_stream_t stream) {
    TG_REQUIRE(T >= 0 && W > 0 && H > 0 && tw > 0 && th > 0, "sizes");
    TG_REQUIRE(tw * th <= 1024, "tile_width * tile_height must be <= 1024");
    TG_REQUIRE(max_layers >= 1, "max_layers must be >= 1");
    TG_REQUIRE(workspace && info_host && offsets && image && depthmap && final_weights && ends, "null pointer");
    TG_REQUIRE(((uintptr_t)workspace & 255) == 0, "workspace must be 256-byte aligned");
    TG_REQUIRE(list_capacity < 0x80000000u, "list capacity must stay below 2^31");
    const int tiles_x = (W + tw - 1) / tw, tiles_y = (H + th - 1) / th;
    const int tiles = tiles_x * tiles_y;
    ForwardWorkspace ws(workspace, T, list_capacity);
    if (workspace_bytes < ws.total) {
        tg_host::set_error("forward workspace: need %zu bytes, got %zu", ws.total, workspace_bytes);
        return TG_ERR_WORKSPACE;
    }
    cudaStream_t s = (cudaStream_t)stream;
    StageTimer timer(stage_ms_host != nullptr, s);
    info_host[0] = 0;
    info_host[1] = 0;

    const int end_bit = 32 + ceil_log2(tiles);
    const int passes = (end_bit + 7) / 8;
    // pick the starting buffers so that the sorted ids land in the caller's array
    uint32_t* ids_a = (passes & 1) ? ws.ids_tmp : (uint32_t*)sorted_ids;
    uint32_t* ids_b = (passes & 1) ? (uint32_t*)sorted_ids : ws.ids_tmp;
    TG_REQUIRE(list_capacity == 0 || sorted_ids != nullptr, "null sorted_ids");
    cudaEvent_t k_ready;
    if (int st = scratch_event(&k_ready)) return st;

    timer.mark();                                                    // [0] start of "init"
    // error word, scan tickets and look-back words, and the sort's look-back words, tickets and digit
    // counters (sized for the whole list capacity): one clear
    const size_t clear = (size_t)((char*)ws.sort_scratch - (char*)ws.status) +
                         (list_capacity > 0 ? tg_host::sort_scratch_clear_bytes(list_capacity, passes) : 0);
    TG_CUDA(cudaMemsetAsync(ws.status, 0, clear, s));
    timer.mark();                                                    // [1] start of "bary_transforms" (preprocess + scan)
    int st = tg_host::preprocess_scan(vertices, indices, colors, opacities, T, W, H, tw, th, tri_geo, tri_attr,
                                      ws.tri_offsets, ws.scan_scratch, ws.status, s);
    if (st) return st;
    timer.mark();                                                    // [2] start of "per_tile_lists"
    TG_CUDA(cudaMemcpyAsync(&info_host[0], ws.tri_offsets + T, sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
    TG_CUDA(cudaEventRecord(k_ready, s));
    // Keys are emitted while K travels to the host: the kernel drops entries beyond the capacity, and
    // nothing that depends on them is launched before K has been checked.
    if (list_capacity > 0) {
        uint32_t* hist = (uint32_t*)ws.sort_scratch;
        uint32_t* ctr = (uint32_t*)((char*)ws.sort_scratch + tg::kHistBytes);
        const tg::HistArgs h = {hist, ctr + tg::kHistDoneWord, 0, end_bit, passes};
        st = tg_host::emit_keys(vertices, indices, T, W, H, tw, th, ws.tri_offsets, ws.keys_a, ids_a, list_capacity, h, s);
        if (st) return st;
    }
    TG_CUDA(cudaEventSynchronize(k_ready));
    const uint32_t K = info_host[0];
    if (K > list_capacity) {
        tg_host::set_error("K = %u exceeds the list capacity %u", K, list_capacity);
        return TG_ERR_CAPACITY;
    }
    timer.mark();                                                    // [3] start of "sorting"
    int in_b = 0;
    st = tg_host::sort_pairs(ws.keys_a, ws.keys_b, ids_a, ids_b, K, 0, end_bit, ws.sort_scratch, ws.sort_scratch_bytes,
                             ws.status, &in_b, true, s);
    if (st) return st;
    st = tg_tile_ranges(in_b ? ws.keys_b : ws.keys_a, K, tiles, offsets, stream);
    if (st) return st;
    timer.mark();                                                    // [4] start of "rasterization"
    st = tg_blend_forward(tri_geo, tri_attr, sorted_ids, offsets, W, H, tw, th, thr, per_pixel_sort, max_layers, image,
                          depthmap, final_weights, ends, selection, stream);
    if (st) return st;
    timer.mark();                                                    // [5] end
    // device error word: valid on the host once the stream has been synchronised
    TG_CUDA(cudaMemcpyAsync(&info_host[1], ws.status, sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
    if (stage_ms_host) {
        TG_CUDA(cudaStreamSynchronize(s));
        float ms[5];
        for (int i = 0; i < 5; i++) TG_CUDA(cudaEventElapsedTime(&ms[i], timer.ev[i], timer.ev[i + 1]));
        stage_ms_host[0] = ms[0];   // init
        stage_ms_host[1] = ms[2];   // per_tile_lists: K read-back + key emission
        stage_ms_host[2] = ms[3];   // sorting: radix sort + tile ranges
        stage_ms_host[3] = ms[1];   // bary_transforms: the fused preprocess + scan kernel
        stage_ms_host[4] = ms[4];   // rasterization
        if (info_host[1]) {
            tg_host::set_error("device error word = %u", info_host[1]);
            return TG_ERR_DEVICE_FLAG;
        }
    }
    return TG_OK;
}

}  // extern "C"
