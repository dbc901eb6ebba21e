// Host <-> device transfer engine behind execute_function: two copy lanes (streams) beside the
// launch stream, fences between them, and a pool of host threads that stages caller memory into
// page-locked memory while the calling thread queues DMAs, launches and read-backs chunk by chunk.
//
// The reference uploads every ndarray argument into its simulated HBM with a flatten() copy and
// reads every one back into a new array (ktir_cpu/interpreter.py:156-194).  Here the same two
// obligations — the device gets the data, the caller gets a fresh array — are met by ONE host
// copy: caller array -> page-locked result array, which is both the array handed back and the
// source of the DMA.  Upload of chunk i+1, kernels of chunk i and read-back of chunk i-1 overlap.
#include <condition_variable>
#include <deque>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#include <emmintrin.h>
#include <sched.h>

#include "common.cuh"

namespace {

// Copy for data that the DMA engine, not this core, reads next: streaming stores keep the
// destination out of the caches (no read-for-ownership, no dirty lines for the DMA to snoop).
void stream_copy(char* dst, const char* src, size_t n) {
    const size_t head = (16 - (reinterpret_cast<uintptr_t>(dst) & 15)) & 15;
    if (n < 256 || head > n) {
        memcpy(dst, src, n);
        return;
    }
    memcpy(dst, src, head);
    dst += head, src += head, n -= head;
    size_t i = 0;
    for (; i + 64 <= n; i += 64) {
        const __m128i a = _mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i));
        const __m128i b = _mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i + 16));
        const __m128i c = _mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i + 32));
        const __m128i d = _mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i + 48));
        _mm_stream_si128(reinterpret_cast<__m128i*>(dst + i), a);
        _mm_stream_si128(reinterpret_cast<__m128i*>(dst + i + 16), b);
        _mm_stream_si128(reinterpret_cast<__m128i*>(dst + i + 32), c);
        _mm_stream_si128(reinterpret_cast<__m128i*>(dst + i + 48), d);
    }
    _mm_sfence();
    if (i < n) memcpy(dst + i, src + i, n - i);
}

// A fixed set of host threads that run batches of numbered tasks.  begin() hands a batch over and
// returns at once; the threads take task numbers in order; end() waits for the batch.
class CopyPool {
public:
    explicit CopyPool(int n) { resize(n); }
    ~CopyPool() { stop(); }

    void resize(int n) {
        stop();
        quit_ = false;
        for (int i = 0; i < n; ++i) threads_.emplace_back([this] { run(); });
    }
    int size() const { return (int)threads_.size(); }

    void begin(int n, std::function<void(int)> fn) {
        std::unique_lock<std::mutex> lk(mu_);
        idle_.wait(lk, [this] { return !busy_; });      // one batch at a time (contexts share the pool)
        busy_ = true;
        fn_ = std::move(fn);
        next_ = 0;
        total_ = n;
        pending_ = n;
        if (threads_.empty()) {                         // no copy threads: the caller does the work here
            lk.unlock();
            for (int i = 0; i < n; ++i) fn_(i);
            lk.lock();
            pending_ = 0;
            return;
        }
        work_.notify_all();
    }
    void end() {
        std::unique_lock<std::mutex> lk(mu_);
        done_.wait(lk, [this] { return pending_ == 0; });
        busy_ = false;
        fn_ = nullptr;
        idle_.notify_one();
    }

private:
    void run() {
        std::unique_lock<std::mutex> lk(mu_);
        for (;;) {
            work_.wait(lk, [this] { return quit_ || (busy_ && next_ < total_); });
            if (quit_) return;
            const int i = next_++;
            lk.unlock();
            fn_(i);
            lk.lock();
            if (--pending_ == 0) done_.notify_all();
        }
    }
    void stop() {
        {
            std::lock_guard<std::mutex> lk(mu_);
            quit_ = true;
        }
        work_.notify_all();
        for (auto& t : threads_) t.join();
        threads_.clear();
    }

    std::mutex mu_;
    std::condition_variable work_, done_, idle_;
    std::vector<std::thread> threads_;
    std::function<void(int)> fn_;
    int next_ = 0, total_ = 0, pending_ = 0;
    bool quit_ = false, busy_ = false;
};

CopyPool& pool() {
    static CopyPool* p = nullptr;          // leaked on purpose: no join during process teardown
    static std::once_flag once;
    std::call_once(once, [] {
        // the CPUs this process may run on (a container or a pinned rank sees fewer than the machine has)
        unsigned hw = std::thread::hardware_concurrency();
        cpu_set_t set;
        if (sched_getaffinity(0, sizeof(set), &set) == 0 && CPU_COUNT(&set) > 0) hw = (unsigned)CPU_COUNT(&set);
        int n = hw >= 16 ? 8 : hw >= 4 ? (int)hw / 2 : 1;
        p = new CopyPool(n);
    });
    return *p;
}

constexpr size_t PIECE_MAX = 1u << 20, PIECE_MIN = 128u << 10;   // host copy granule

int lanes_ready(ktb_ctx* ctx) {
    if (ctx->lanes_ok) return KTB_OK;
    KTB_CUDA(ctx, cudaSetDevice(ctx->device));
    for (int i = 0; i < 2; ++i) KTB_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->lane[i], cudaStreamNonBlocking));
    for (int i = 0; i < KTB_NUM_FENCES; ++i) KTB_CUDA(ctx, cudaEventCreateWithFlags(&ctx->fences[i], cudaEventDisableTiming));
    ctx->lanes_ok = true;
    return KTB_OK;
}

cudaStream_t stream_of(ktb_ctx* ctx, int which) { return which == 0 ? ctx->stream : ctx->lane[which - 1]; }

int fence(ktb_ctx* ctx, int from, int to) {
    cudaEvent_t ev = ctx->fences[ctx->next_fence++ % KTB_NUM_FENCES];
    KTB_CUDA(ctx, cudaEventRecord(ev, stream_of(ctx, from)));
    KTB_CUDA(ctx, cudaStreamWaitEvent(stream_of(ctx, to), ev, 0));
    return KTB_OK;
}

int copy_region(ktb_ctx* ctx, void* dst, const void* src, const ktb_region& r, cudaMemcpyKind kind, cudaStream_t st) {
    if (r.width == 0 || r.height == 0) return KTB_OK;
    if (r.height == 1 || r.pitch == r.width)
        KTB_CUDA(ctx, cudaMemcpyAsync(dst, src, r.width * r.height, kind, st));
    else
        KTB_CUDA(ctx, cudaMemcpy2DAsync(dst, r.pitch, src, r.pitch, r.width, r.height, kind, st));
    return KTB_OK;
}

struct Piece {          // part of one upload region: rows [r0, r0 + rows) x bytes [x0, x0 + len)
    char* dst;
    const char* src;
    size_t len, rows, pitch;
    int chunk;
};

// A queued ktb_run_pipeline call with everything it points at copied, so that the caller may move on.
struct Job {
    void* arena;
    std::vector<ktb_pipe_chunk> chunks;
    std::vector<std::vector<ktb_region>> up, down;
    std::vector<void*> pinned;
    std::vector<const void*> src;
    ktb_status* snapshot;
    int event_slot, event_lane;
    uint64_t seq;
};

}  // namespace

extern "C" int ktb_run_pipeline(ktb_ctx*, void*, const ktb_pipe_chunk*, int, void* const*, const void* const*, int);
extern "C" int ktb_status_snapshot(ktb_ctx*, ktb_status*);
extern "C" int ktb_event_record_on(ktb_ctx*, int, int);

// One thread per context that issues queued jobs in order, so that the host thread that prepared a
// call can prepare the next one while this one is staged and queued on the device.
struct ktb_submitter {
    std::mutex mu;
    std::condition_variable work, progress;
    std::deque<Job> queue;
    std::thread thread;
    uint64_t next_seq = 1, done_seq = 0;
    int first_error = KTB_OK;
    uint64_t error_seq = 0;
    bool quit = false;

    void run(ktb_ctx* ctx) {
        cudaSetDevice(ctx->device);
        std::unique_lock<std::mutex> lk(mu);
        for (;;) {
            work.wait(lk, [this] { return quit || !queue.empty(); });
            if (queue.empty()) return;
            Job job = std::move(queue.front());
            queue.pop_front();
            lk.unlock();
            for (size_t c = 0; c < job.chunks.size(); ++c) {
                job.chunks[c].up = job.up[c].data();
                job.chunks[c].down = job.down[c].data();
            }
            int rc = ktb_run_pipeline(ctx, job.arena, job.chunks.data(), (int)job.chunks.size(), job.pinned.data(),
                                      job.src.data(), (int)job.pinned.size());
            if (rc == KTB_OK && job.snapshot) rc = ktb_status_snapshot(ctx, job.snapshot);
            if (rc == KTB_OK && job.event_slot >= 0) {
                // behind the read-backs when there are any, else behind the launches
                if (job.event_lane == 2) rc = fence(ctx, 0, 2);
                if (rc == KTB_OK) rc = ktb_event_record_on(ctx, job.event_slot, job.event_lane);
            }
            lk.lock();
            if (rc != KTB_OK && first_error == KTB_OK) first_error = rc, error_seq = job.seq;
            done_seq = job.seq;
            progress.notify_all();
        }
    }
};

void ktb_transfer_destroy(ktb_ctx* ctx) {
    if (ctx->submitter) {
        {
            std::lock_guard<std::mutex> lk(ctx->submitter->mu);
            ctx->submitter->quit = true;
        }
        ctx->submitter->work.notify_all();
        ctx->submitter->thread.join();
        delete ctx->submitter;
        ctx->submitter = nullptr;
    }
    if (!ctx->lanes_ok) return;
    for (int i = 0; i < 2; ++i) {
        cudaStreamSynchronize(ctx->lane[i]);
        cudaStreamDestroy(ctx->lane[i]);
    }
    for (int i = 0; i < KTB_NUM_FENCES; ++i) cudaEventDestroy(ctx->fences[i]);
    ctx->lanes_ok = false;
}

// Everything queued with ktb_submit_pipeline has been issued to the device (0 = all jobs so far).
int ktb_transfer_drain(ktb_ctx* ctx, uint64_t seq) {
    ktb_submitter* s = ctx->submitter;
    if (!s) return KTB_OK;
    std::unique_lock<std::mutex> lk(s->mu);
    const uint64_t want = seq ? seq : s->next_seq - 1;
    s->progress.wait(lk, [&] { return s->done_seq >= want; });
    if (s->first_error != KTB_OK && s->error_seq <= want) {
        const int rc = s->first_error;
        s->first_error = KTB_OK;
        return rc;
    }
    return KTB_OK;
}

int ktb_transfer_sync(ktb_ctx* ctx) {
    if (int rc = ktb_transfer_drain(ctx, 0)) return rc;
    if (!ctx->lanes_ok || !ctx->lanes_used) return KTB_OK;
    for (int i = 0; i < 2; ++i) KTB_CUDA(ctx, cudaStreamSynchronize(ctx->lane[i]));
    ctx->lanes_used = false;
    return KTB_OK;
}

extern "C" {

int ktb_set_copy_threads(int n) {
    if (n < 0 || n > 64) return KTB_E_ARG;
    pool().resize(n);
    return KTB_OK;
}

int ktb_copy_threads(void) { return pool().size(); }

int ktb_lane_fence(ktb_ctx* ctx, int from, int to) {
    if (!ctx || from < 0 || from > 2 || to < 0 || to > 2 || from == to) return KTB_E_ARG;
    if (int rc = lanes_ready(ctx)) return rc;
    ctx->lanes_used = true;
    return fence(ctx, from, to);
}

int ktb_lane_d2h(ktb_ctx* ctx, void* host_dst, const void* dev_src, size_t width, size_t height, size_t pitch) {
    if (!ctx) return KTB_E_ARG;
    if (int rc = lanes_ready(ctx)) return rc;
    ctx->lanes_used = true;
    ktb_region r{};
    r.width = width, r.height = height, r.pitch = pitch;
    return copy_region(ctx, host_dst, dev_src, r, cudaMemcpyDeviceToHost, ctx->lane[1]);
}

int ktb_submit_pipeline(ktb_ctx* ctx, void* arena, const ktb_pipe_chunk* chunks, int n_chunks, void* const* pinned,
                        const void* const* src, int n_tensors, ktb_status* snapshot, int event_slot, uint64_t* seq_out) {
    if (!ctx || !chunks || n_chunks < 0 || !seq_out || event_slot >= KTB_NUM_EVENTS) return KTB_E_ARG;
    if (int rc = lanes_ready(ctx)) return rc;
    if (!ctx->submitter) {
        ctx->submitter = new ktb_submitter();
        ctx->submitter->thread = std::thread([ctx] { ctx->submitter->run(ctx); });
    }
    Job job;
    job.arena = arena;
    job.chunks.assign(chunks, chunks + n_chunks);
    bool reads_back = false;
    for (int c = 0; c < n_chunks; ++c) {
        job.up.emplace_back(chunks[c].up, chunks[c].up + chunks[c].n_up);
        job.down.emplace_back(chunks[c].down, chunks[c].down + chunks[c].n_down);
        reads_back = reads_back || chunks[c].n_down > 0;
    }
    job.pinned.assign(pinned, pinned + n_tensors);
    job.src.assign(src, src + n_tensors);
    job.snapshot = snapshot;
    job.event_slot = event_slot;
    job.event_lane = reads_back ? 2 : 0;
    ktb_submitter* s = ctx->submitter;
    {
        std::lock_guard<std::mutex> lk(s->mu);
        job.seq = s->next_seq++;
        *seq_out = job.seq;
        s->queue.push_back(std::move(job));
    }
    s->work.notify_one();
    return KTB_OK;
}

int ktb_wait_submitted(ktb_ctx* ctx, uint64_t seq) {
    if (!ctx) return KTB_E_ARG;
    return ktb_transfer_drain(ctx, seq);
}

int ktb_run_pipeline(ktb_ctx* ctx, void* arena, const ktb_pipe_chunk* chunks, int n_chunks, void* const* pinned,
                     const void* const* src, int n_tensors) {
    if (!ctx || !chunks || n_chunks < 0 || (n_tensors > 0 && (!pinned || !src))) return KTB_E_ARG;
    if (int rc = lanes_ready(ctx)) return rc;
    KTB_CUDA(ctx, cudaSetDevice(ctx->device));
    ctx->lanes_used = true;
    char* base = static_cast<char*>(arena);

    // every upload region cut into pieces, in chunk order; a region whose source already is its
    // page-locked array needs no host copy
    // (small calls get small pieces, so that a few MB still spread over the copy threads)
    size_t staged = 0;
    for (int c = 0; c < n_chunks; ++c)
        for (int k = 0; k < chunks[c].n_up; ++k) staged += chunks[c].up[k].width * chunks[c].up[k].height;
    size_t PIECE = staged / (2 * (size_t)(pool().size() > 0 ? pool().size() : 1));
    PIECE = PIECE < PIECE_MIN ? PIECE_MIN : PIECE > PIECE_MAX ? PIECE_MAX : (PIECE + 4095) & ~(size_t)4095;
    std::vector<Piece> pieces;
    std::vector<int> left(n_chunks, 0);
    for (int c = 0; c < n_chunks; ++c) {
        for (int k = 0; k < chunks[c].n_up; ++k) {
            const ktb_region& r = chunks[c].up[k];
            if (r.tensor < 0 || r.tensor >= n_tensors) return ktb_fail(ctx, KTB_E_ARG, "ktb_run_pipeline", "bad tensor index");
            char* dst = static_cast<char*>(pinned[r.tensor]) + r.rel;
            const char* from = static_cast<const char*>(src[r.tensor]) + r.rel;
            if (dst == from || r.width == 0 || r.height == 0) continue;
            if (r.height == 1 || r.pitch == r.width) {
                const size_t total = r.width * r.height;
                for (size_t off = 0; off < total; off += PIECE)
                    pieces.push_back({dst + off, from + off, off + PIECE <= total ? PIECE : total - off, 1, 0, c});
            } else {
                size_t band = PIECE / r.width;
                if (band < 1) band = 1;
                for (size_t r0 = 0; r0 < r.height; r0 += band)
                    pieces.push_back({dst + r0 * r.pitch, from + r0 * r.pitch, (size_t)r.width,
                                      r0 + band <= r.height ? band : (size_t)r.height - r0, (size_t)r.pitch, c});
            }
        }
    }
    for (const Piece& p : pieces) ++left[p.chunk];

    std::mutex mu;
    std::condition_variable cv;
    const bool any = !pieces.empty();
    if (any)
        pool().begin((int)pieces.size(), [&](int i) {
            const Piece& p = pieces[i];
            if (p.rows == 1) stream_copy(p.dst, p.src, p.len);
            else
                for (size_t r = 0; r < p.rows; ++r) stream_copy(p.dst + r * p.pitch, p.src + r * p.pitch, p.len);
            std::lock_guard<std::mutex> lk(mu);
            if (--left[p.chunk] == 0) cv.notify_all();
        });

    int rc = KTB_OK;
    for (int c = 0; c < n_chunks && rc == KTB_OK; ++c) {
        const ktb_pipe_chunk& ch = chunks[c];
        {
            std::unique_lock<std::mutex> lk(mu);
            cv.wait(lk, [&] { return left[c] == 0; });       // this chunk's data is in page-locked memory
        }
        for (int k = 0; k < ch.n_up && rc == KTB_OK; ++k) {
            const ktb_region& r = ch.up[k];
            if (r.dev_off == KTB_NO_DEVICE) continue;         // the caller's copy only
            rc = copy_region(ctx, base + r.dev_off, static_cast<char*>(pinned[r.tensor]) + r.rel, r,
                             cudaMemcpyHostToDevice, ctx->lane[0]);
        }
        if (rc == KTB_OK && ch.n_up > 0) rc = fence(ctx, 1, 0);
        if (rc == KTB_OK && ch.launch) rc = ch.launch(ctx, ch.launch_args);
        if (rc == KTB_OK && ch.n_down > 0) rc = fence(ctx, 0, 2);
        for (int k = 0; k < ch.n_down && rc == KTB_OK; ++k) {
            const ktb_region& r = ch.down[k];
            if (r.tensor < 0 || r.tensor >= n_tensors) rc = ktb_fail(ctx, KTB_E_ARG, "ktb_run_pipeline", "bad tensor index");
            else rc = copy_region(ctx, static_cast<char*>(pinned[r.tensor]) + r.rel, base + r.dev_off, r,
                                  cudaMemcpyDeviceToHost, ctx->lane[1]);
        }
    }
    if (any) pool().end();        // (on an error: the copy threads still finish their batch before `pieces` goes away)
    return rc;
}

}  // extern "C"
