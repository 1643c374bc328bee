// Raw tensor files (reference: ioutils.cu:3-45): device buffer <-> file through a
// host bounce buffer; byte counts are 32-bit as in the reference.
#include "ioutils.cuh"

#include <cstdio>
#include <stdexcept>
#include <vector>

#include "zkllm_ext.hpp"

void savebin(const string& filename, const void* gpudata, uint size) {
    std::vector<char> host(size);
    if (size) zkllm::check(zkb_memcpy_d2h(host.data(), gpudata, size, nullptr));
    FILE* f = fopen(filename.c_str(), "wb");
    if (!f) throw std::runtime_error("savebin: cannot open " + filename);
    const size_t wrote = fwrite(host.data(), 1, size, f);
    fclose(f);
    if (wrote != size) throw std::runtime_error("savebin: short write to " + filename);
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
    std::vector<char> host(size);
    FILE* f = fopen(filename.c_str(), "rb");
    if (!f) throw std::runtime_error("loadbin: cannot open " + filename);
    const size_t got = fread(host.data(), 1, size, f);
    fclose(f);
    if (got != size) throw std::runtime_error("loadbin: short read from " + filename);
    if (size) zkllm::check(zkb_memcpy_h2d(gpudata, host.data(), size, nullptr));
}
