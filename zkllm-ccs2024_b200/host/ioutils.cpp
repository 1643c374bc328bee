// Raw tensor files (reference: ioutils.cu:3-45): device buffer <-> file, byte
// counts 32-bit as in the reference.  The reference stages the whole file in a
// pageable buffer; here two page-locked 16 MiB buffers alternate, so reading (or
// writing) a chunk overlaps the DMA of its neighbour.
//
// Resident files (no counterpart in the reference, off by default): a process that runs many
// stages - `zkllm-driver batch` - can keep a device copy of every file it loads or saves
// (zkllm::set_resident_files).  A later loadbin of the same file is then a device-to-device copy:
// generators, weights and commitments are read from disk once per process, and an activation
// saved by one stage is already on the device when the next stage loads it.  Every file is still
// written and a cached copy is used only while the file's size, inode and modification time are
// those seen when the copy was made, so files rewritten by another program are read again.
//
// Deferred writes (no counterpart in the reference, off by default; zkllm::set_deferred_saves): savebin copies the
// tensor into a page-locked host buffer (one DMA) and hands the buffer to a writer thread, so the 5 to 10 ms that a
// 32 MiB file takes to reach the page cache pass while the caller is already proving.  A file is complete once
// zkllm::flush_saves() has returned (`zkllm-driver batch` calls it before it answers a line), and loadbin / findsize
// of a file that is still being written wait for it first.  A failed write is reported by the call that waits.
// These functions are for one host thread at a time, like the rest of the class library.
#include "ioutils.cuh"

#include <sys/stat.h>

#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <deque>
#include <exception>
#include <list>
#include <map>
#include <mutex>
#include <stdexcept>
#include <thread>
#include <vector>

#include "zkllm_ext.hpp"

namespace {

struct FileId {
    off_t size = 0;
    ino_t ino = 0;
    long long mtime_ns = 0;
    bool operator==(const FileId& o) const { return size == o.size && ino == o.ino && mtime_ns == o.mtime_ns; }
};
bool file_id(const string& name, FileId* id) {
    struct stat st;
    if (stat(name.c_str(), &st) != 0) return false;
    id->size = st.st_size;
    id->ino = st.st_ino;
    id->mtime_ns = (long long)st.st_mtim.tv_sec * 1000000000LL + st.st_mtim.tv_nsec;
    return true;
}

struct Resident {
    FileId id;
    void* dev = nullptr;
    size_t bytes = 0;
    std::list<string>::iterator age;     // position in the least-recently-used list
};
struct ResidentFiles {
    bool on = false;
    size_t limit = (size_t)24 << 30, used = 0;
    std::map<string, Resident> files;
    std::list<string> lru;               // front = most recently used
    zkllm::ResidentStats stats;

    void drop(const string& name) {
        auto it = files.find(name);
        if (it == files.end()) return;
        zkb_free_default_stream(it->second.dev);
        used -= it->second.bytes;
        lru.erase(it->second.age);
        files.erase(it);
    }
    // keeps a device copy of `bytes` bytes at d_src as the content of `name` (as it is on disk now; with
    // `written_later` the file is still on its way to the disk and confirm() completes the entry)
    void remember(const string& name, const void* d_src, size_t bytes, bool written_later = false) {
        drop(name);
        FileId id;
        if (bytes > limit) return;
        if (!written_later && (!file_id(name, &id) || (size_t)id.size != bytes)) return;
        while (used + bytes > limit && !lru.empty()) drop(lru.back());
        void* p = nullptr;
        if (zkb_malloc(&p, bytes) != ZKB_OK) return;          // no room: simply not cached
        if (zkb_memcpy_d2d(p, d_src, bytes, nullptr) != ZKB_OK || zkb_sync(nullptr) != ZKB_OK) { zkb_free_default_stream(p); return; }
        lru.push_front(name);
        Resident r;
        r.id = id; r.dev = p; r.bytes = bytes; r.age = lru.begin();
        files[name] = r;
        used += bytes;
    }
    // the deferred write of `name` has finished: take the file's identity now
    void confirm(const string& name) {
        auto it = files.find(name);
        if (it == files.end()) return;
        FileId id;
        if (!file_id(name, &id) || (size_t)id.size != it->second.bytes) drop(name);
        else it->second.id = id;
    }
    // copies the cached content of `name` to d_dst when the file is unchanged since it was cached
    bool recall(const string& name, void* d_dst, size_t bytes) {
        auto it = files.find(name);
        if (it == files.end()) return false;
        FileId now;
        if (!file_id(name, &now) || !(now == it->second.id) || it->second.bytes != bytes) {
            drop(name);
            return false;
        }
        zkllm::check(zkb_memcpy_d2d(d_dst, it->second.dev, bytes, nullptr));
        zkllm::check(zkb_sync(nullptr));
        lru.splice(lru.begin(), lru, it->second.age);
        return true;
    }
};
ResidentFiles& resident() {
    static ResidentFiles r;
    return r;
}

constexpr size_t kChunk = 16u << 20;

// ---- deferred writes ---------------------------------------------------------------------
struct WriteJob {
    string name;
    char* buf = nullptr;        // page-locked, from the buffer pool below
    size_t cap = 0, bytes = 0;
};
struct Writer {
    bool on = false;
    std::mutex mu;
    std::condition_variable wake, idle;
    std::deque<WriteJob> queue;
    std::map<string, unsigned> in_flight;            // file -> jobs queued or being written
    std::map<string, string> failed;                 // file -> what went wrong
    std::vector<std::pair<char*, size_t>> free_bufs; // page-locked buffers waiting for reuse
    size_t buffers = 0;
    std::thread thread;
    bool quit = false;

    void run() {
        std::unique_lock<std::mutex> lk(mu);
        for (;;) {
            wake.wait(lk, [&] { return quit || !queue.empty(); });
            if (queue.empty()) return;
            WriteJob job = queue.front();
            queue.pop_front();
            lk.unlock();
            string err;
            FILE* f = fopen(job.name.c_str(), "wb");
            if (!f) err = "savebin: cannot open " + job.name;
            else {
                setvbuf(f, nullptr, _IONBF, 0);
                if (fwrite(job.buf, 1, job.bytes, f) != job.bytes) err = "savebin: short write to " + job.name;
                if (fclose(f) != 0 && err.empty()) err = "savebin: cannot close " + job.name;
            }
            lk.lock();
            if (!err.empty()) failed[job.name] = err;
            free_bufs.push_back({job.buf, job.cap});
            if (--in_flight[job.name] == 0) in_flight.erase(job.name);
            idle.notify_all();
        }
    }
    ~Writer() {
        {
            std::lock_guard<std::mutex> lk(mu);
            quit = true;
        }
        wake.notify_all();
        if (thread.joinable()) thread.join();      // drains the queue first: run() leaves only when it is empty
    }
};
Writer& writer() {
    static Writer w;
    return w;
}
// waits until `name` (every file when name is null) is on disk; throws what its write reported
void wait_written(const string* name) {
    Writer& w = writer();
    std::vector<string> done;
    string err;
    {
        std::unique_lock<std::mutex> lk(w.mu);
        if (w.in_flight.empty() && w.failed.empty()) return;
        w.idle.wait(lk, [&] { return name ? !w.in_flight.count(*name) : w.in_flight.empty(); });
        if (name) {
            auto it = w.failed.find(*name);
            if (it != w.failed.end()) { err = it->second; w.failed.erase(it); }
        } else if (!w.failed.empty()) {
            err = w.failed.begin()->second;
            w.failed.clear();
        }
    }
    if (!err.empty()) throw std::runtime_error(err);
}

// process-wide staging buffers, allocated on first use and kept
char* staging(int which) {
    static char* buf[2] = {nullptr, nullptr};
    if (!buf[which]) {
        void* p = nullptr;
        zkllm::check(zkb_host_alloc(&p, kChunk));
        buf[which] = static_cast<char*>(p);
    }
    return buf[which];
}

struct File {
    FILE* f;
    File(const string& name, const char* mode, const char* who) : f(fopen(name.c_str(), mode)) {
        if (!f) throw std::runtime_error(string(who) + ": cannot open " + name);
        setvbuf(f, nullptr, _IONBF, 0);
    }
    ~File() { if (f) fclose(f); }
};

}  // namespace

namespace zkllm {
void set_resident_files(bool on, size_t limit_bytes) {
    ResidentFiles& r = resident();
    r.on = on;
    if (limit_bytes) r.limit = limit_bytes;
    if (!on)
        while (!r.lru.empty()) r.drop(r.lru.back());
}
ResidentStats resident_stats() { return resident().stats; }
}  // namespace zkllm

namespace {
std::vector<string> g_unconfirmed;    // files handed to the writer whose cache entries still lack an identity
void confirm_written(const string* name) {
    wait_written(name);
    ResidentFiles& r = resident();
    for (size_t i = 0; i < g_unconfirmed.size();) {
        if (!name || g_unconfirmed[i] == *name) {
            r.confirm(g_unconfirmed[i]);
            g_unconfirmed[i] = g_unconfirmed.back();
            g_unconfirmed.pop_back();
        } else {
            ++i;
        }
    }
}
}  // namespace

namespace zkllm {
void set_deferred_saves(bool on) {
    if (!on) flush_saves();
    writer().on = on;
}
void flush_saves() { confirm_written(nullptr); }
}  // namespace zkllm

void savebin(const string& filename, const void* gpudata, uint size) {
    Writer& w = writer();
    if (w.on && size) {
        confirm_written(&filename);               // an earlier write of the same file goes first
        WriteJob job;
        job.name = filename;
        job.bytes = size;
        {
            std::unique_lock<std::mutex> lk(w.mu);
            for (;;) {
                for (size_t i = 0; i < w.free_bufs.size(); ++i)
                    if (w.free_bufs[i].second >= size) {
                        job.buf = w.free_bufs[i].first;
                        job.cap = w.free_bufs[i].second;
                        w.free_bufs.erase(w.free_bufs.begin() + i);
                        break;
                    }
                if (job.buf || w.buffers < 8) break;
                if (!w.free_bufs.empty()) {               // all too small: give one back and allocate a larger one
                    zkb_host_free(w.free_bufs.back().first);
                    w.free_bufs.pop_back();
                    --w.buffers;
                    break;
                }
                w.idle.wait(lk);                          // eight buffers are with the writer: wait for one
            }
            if (!job.buf) ++w.buffers;
        }
        if (!job.buf) {
            void* p = nullptr;
            job.cap = ((size_t)size + (kChunk - 1)) / kChunk * kChunk;
            zkllm::check(zkb_host_alloc(&p, job.cap));
            job.buf = static_cast<char*>(p);
        }
        zkllm::check(zkb_memcpy_d2h_async(job.buf, gpudata, size, nullptr));
        zkllm::check(zkb_sync(nullptr));
        ResidentFiles& r = resident();
        if (r.on) {
            r.remember(filename, gpudata, size, true);
            r.stats.saved_files += 1;
            g_unconfirmed.push_back(filename);
        }
        {
            std::lock_guard<std::mutex> lk(w.mu);
            if (!w.thread.joinable()) w.thread = std::thread([&w] { w.run(); });
            w.in_flight[filename] += 1;
            w.queue.push_back(job);
        }
        w.wake.notify_one();
        return;
    }
    {
        File file(filename, "wb", "savebin");
        const char* src = static_cast<const char*>(gpudata);
        // chunk i travels to buffer i & 1 while chunk i - 1 is written out
        size_t prev = 0;
        for (size_t off = 0, i = 0; off < size || prev; off += kChunk, ++i) {
            const size_t len = off < size ? (size - off < kChunk ? size - off : kChunk) : 0;
            if (len) zkllm::check(zkb_memcpy_d2h_async(staging(i & 1), src + off, len, nullptr));
            if (prev && fwrite(staging((i + 1) & 1), 1, prev, file.f) != prev)
                throw std::runtime_error("savebin: short write to " + filename);
            if (len) zkllm::check(zkb_sync(nullptr));
            prev = len;
        }
    }   // closed: size and modification time are final
    ResidentFiles& r = resident();
    if (r.on) {
        r.remember(filename, gpudata, size);
        r.stats.saved_files += 1;
    }
}

uint findsize(const string& filename) {
    confirm_written(&filename);
    FILE* f = fopen(filename.c_str(), "rb");
    if (!f) throw std::runtime_error("findsize: cannot open " + filename);
    fseek(f, 0, SEEK_END);
    const uint size = (uint)ftell(f);
    fclose(f);
    return size;
}

void loadbin(const string& filename, void* gpudata, uint size) {
    confirm_written(&filename);
    ResidentFiles& r = resident();
    if (r.on && r.recall(filename, gpudata, size)) {
        r.stats.loads_from_device += 1;
        r.stats.bytes_from_device += size;
        return;
    }
    if (r.on) {
        r.stats.loads_from_disk += 1;
        r.stats.bytes_from_disk += size;
    }
    {
        File file(filename, "rb", "loadbin");
    char* dst = static_cast<char*>(gpudata);
    for (size_t off = 0, i = 0; off < size; off += kChunk, ++i) {
        const size_t len = size - off < kChunk ? size - off : kChunk;
        // reading chunk i overlaps the copy of chunk i - 1, issued from the other buffer
        if (fread(staging(i & 1), 1, len, file.f) != len) throw std::runtime_error("loadbin: short read from " + filename);
        zkllm::check(zkb_sync(nullptr));
        zkllm::check(zkb_memcpy_h2d_async(dst + off, staging(i & 1), len, nullptr));
    }
    zkllm::check(zkb_sync(nullptr));
    }
    if (r.on) r.remember(filename, gpudata, size);
}
