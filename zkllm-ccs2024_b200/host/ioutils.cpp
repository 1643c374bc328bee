// Raw tensor files (reference: ioutils.cu:3-45): device buffer <-> file, byte
// counts 32-bit as in the reference.  The reference stages the whole file in a
// pageable buffer; here two page-locked 16 MiB buffers alternate, so reading (or
// writing) a chunk overlaps the DMA of its neighbour.
#include "ioutils.cuh"

#include <cstdio>
#include <stdexcept>

#include "zkllm_ext.hpp"

namespace {

constexpr size_t kChunk = 16u << 20;

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

void savebin(const string& filename, const void* gpudata, uint size) {
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
}

uint findsize(const string& filename) {
    FILE* f = fopen(filename.c_str(), "rb");
    if (!f) throw std::runtime_error("findsize: cannot open " + filename);
    fseek(f, 0, SEEK_END);
    const uint size = (uint)ftell(f);
    fclose(f);
    return size;
}

void loadbin(const string& filename, void* gpudata, uint size) {
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
