// Optimizer-state checkpoint (rlcu_checkpoint_* in include/rlcu_adamw.h).
// RL.cu only has a stub here (include/training/trainer.h:317-319); the format
// is this library's own.  Host I/O plus staged device copies; no kernels.
#include "rlcu_adamw.h"

#include <unistd.h>

#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "host_util.h"

namespace {

using rlcu::set_error;

constexpr char kMagic[8] = {'R', 'L', 'C', 'U', 'O', 'P', 'T', '1'};
constexpr size_t kStage = 64u << 20;   // bytes per staged copy

struct Header {               // 128 bytes on disk
    char magic[8];
    uint32_t version;
    uint32_t header_bytes;
    rlcu_checkpoint_info info;
    unsigned char pad[128 - 16 - sizeof(rlcu_checkpoint_info)];
};
static_assert(sizeof(Header) == 128, "checkpoint header is 128 bytes");

inline uint64_t fnv1a(uint64_t h, const unsigned char* p, size_t n) {
    for (size_t i = 0; i < n; i++) {
        h ^= p[i];
        h *= 1099511628211ull;
    }
    return h;
}

struct File {
    FILE* f = nullptr;
    ~File() { if (f) fclose(f); }
};

int read_header(FILE* f, const char* path, Header* h) {
    if (fread(h, sizeof(Header), 1, f) != 1) return set_error(RLCU_ERR_INVALID, "%s: too short for a checkpoint header", path);
    if (memcmp(h->magic, kMagic, 8) != 0) return set_error(RLCU_ERR_INVALID, "%s: not an optimizer checkpoint (bad magic)", path);
    if (h->version != 1 || h->header_bytes != sizeof(Header))
        return set_error(RLCU_ERR_UNSUPPORTED, "%s: checkpoint version %u is not supported", path, h->version);
    return RLCU_OK;
}

}  // namespace

extern "C" {

int rlcu_checkpoint_save(const char* path, const rlcu_checkpoint_info* info,
                         const float* m, const float* v, const float* master, void* stream) {
    if (!path || !info) return set_error(RLCU_ERR_INVALID, "null path or info");
    if (info->state_elems && (!m || !v)) return set_error(RLCU_ERR_INVALID, "null state arrays");
    if ((info->has_master != 0) != (master != nullptr) && info->state_elems)
        return set_error(RLCU_ERR_INVALID, "has_master does not match the master pointer");
    // Written beside the target and renamed over it once complete and on disk, so a crash
    // or a full disk in mid-save leaves the previous checkpoint as it was.
    const std::string tmp = std::string(path) + ".tmp";
    struct Cleanup {                        // removes the partial file on every early return
        const std::string& name;
        bool armed = false;
        ~Cleanup() { if (armed) remove(name.c_str()); }
    } cleanup{tmp};
    File out;
    out.f = fopen(tmp.c_str(), "wb");
    if (!out.f) return set_error(RLCU_ERR_INVALID, "cannot open %s for writing", tmp.c_str());
    cleanup.armed = true;
    Header h;
    memset(&h, 0, sizeof(h));
    memcpy(h.magic, kMagic, 8);
    h.version = 1;
    h.header_bytes = sizeof(Header);
    h.info = *info;
    if (fwrite(&h, sizeof(h), 1, out.f) != 1) return set_error(RLCU_ERR_INVALID, "write to %s failed", tmp.c_str());

    cudaStream_t s = (cudaStream_t)stream;
    std::vector<unsigned char> stage(kStage);
    uint64_t sum = 14695981039346656037ull;
    const float* arrays[3] = {m, v, master};
    for (int a = 0; a < (info->has_master ? 3 : 2); a++) {
        const size_t bytes = (size_t)info->state_elems * sizeof(float);
        for (size_t off = 0; off < bytes; off += kStage) {
            const size_t n = bytes - off < kStage ? bytes - off : kStage;
            RLCU_CUDA(cudaMemcpyAsync(stage.data(), reinterpret_cast<const char*>(arrays[a]) + off, n,
                                      cudaMemcpyDeviceToHost, s));
            RLCU_CUDA(cudaStreamSynchronize(s));
            sum = fnv1a(sum, stage.data(), n);
            if (fwrite(stage.data(), 1, n, out.f) != n) return set_error(RLCU_ERR_INVALID, "write to %s failed", tmp.c_str());
        }
    }
    if (fwrite(&sum, sizeof(sum), 1, out.f) != 1 || fflush(out.f) != 0 || fsync(fileno(out.f)) != 0)
        return set_error(RLCU_ERR_INVALID, "write to %s failed", tmp.c_str());
    FILE* f = out.f;
    out.f = nullptr;
    if (fclose(f) != 0) return set_error(RLCU_ERR_INVALID, "closing %s failed", tmp.c_str());
    if (rename(tmp.c_str(), path) != 0) return set_error(RLCU_ERR_INVALID, "cannot rename %s to %s", tmp.c_str(), path);
    cleanup.armed = false;
    return RLCU_OK;
}

int rlcu_checkpoint_peek(const char* path, rlcu_checkpoint_info* info_out) {
    if (!path || !info_out) return set_error(RLCU_ERR_INVALID, "null path or info");
    File in;
    in.f = fopen(path, "rb");
    if (!in.f) return set_error(RLCU_ERR_INVALID, "cannot open %s", path);
    Header h;
    const int rc = read_header(in.f, path, &h);
    if (rc) return rc;
    *info_out = h.info;
    return RLCU_OK;
}

int rlcu_checkpoint_load(const char* path, rlcu_checkpoint_info* info_out,
                         float* m, float* v, float* master, uint64_t capacity_elems, void* stream) {
    if (!path) return set_error(RLCU_ERR_INVALID, "null path");
    File in;
    in.f = fopen(path, "rb");
    if (!in.f) return set_error(RLCU_ERR_INVALID, "cannot open %s", path);
    Header h;
    int rc = read_header(in.f, path, &h);
    if (rc) return rc;
    const rlcu_checkpoint_info& info = h.info;
    if (info.state_elems > capacity_elems)
        return set_error(RLCU_ERR_INVALID, "%s holds %llu state elements, the buffers only %llu", path,
                         (unsigned long long)info.state_elems, (unsigned long long)capacity_elems);
    if ((info.has_master != 0) != (master != nullptr) && info.state_elems)
        return set_error(RLCU_ERR_INVALID, "%s %s a master copy but the caller %s one", path,
                         info.has_master ? "has" : "lacks", master ? "passed" : "did not pass");
    if (info.state_elems && (!m || !v)) return set_error(RLCU_ERR_INVALID, "null state arrays");

    // First pass, host only: length and checksum.  Nothing is copied into the caller's
    // live state until the whole file is known to be good.
    std::vector<unsigned char> stage(kStage);
    const int n_arrays = info.has_master ? 3 : 2;
    const size_t bytes = (size_t)info.state_elems * sizeof(float);
    uint64_t sum = 14695981039346656037ull;
    for (int a = 0; a < n_arrays; a++) {
        for (size_t off = 0; off < bytes; off += kStage) {
            const size_t n = bytes - off < kStage ? bytes - off : kStage;
            if (fread(stage.data(), 1, n, in.f) != n) return set_error(RLCU_ERR_INVALID, "%s is truncated", path);
            sum = fnv1a(sum, stage.data(), n);
        }
    }
    uint64_t stored = 0;
    if (fread(&stored, sizeof(stored), 1, in.f) != 1) return set_error(RLCU_ERR_INVALID, "%s is truncated (no checksum)", path);
    if (stored != sum) return set_error(RLCU_ERR_INVALID, "%s: checksum mismatch, nothing was loaded", path);

    // Second pass: the copy.  The checksum is taken again in case the file changed in between.
    if (fseek(in.f, (long)sizeof(Header), SEEK_SET) != 0) return set_error(RLCU_ERR_INVALID, "cannot rewind %s", path);
    cudaStream_t s = (cudaStream_t)stream;
    float* arrays[3] = {m, v, master};
    uint64_t sum2 = 14695981039346656037ull;
    for (int a = 0; a < n_arrays; a++) {
        for (size_t off = 0; off < bytes; off += kStage) {
            const size_t n = bytes - off < kStage ? bytes - off : kStage;
            if (fread(stage.data(), 1, n, in.f) != n) return set_error(RLCU_ERR_INVALID, "%s changed while it was read", path);
            sum2 = fnv1a(sum2, stage.data(), n);
            RLCU_CUDA(cudaMemcpyAsync(reinterpret_cast<char*>(arrays[a]) + off, stage.data(), n,
                                      cudaMemcpyHostToDevice, s));
            RLCU_CUDA(cudaStreamSynchronize(s));
        }
    }
    if (sum2 != sum) return set_error(RLCU_ERR_INVALID, "%s changed while it was read; the loaded state is corrupt", path);
    if (info_out) *info_out = info;
    return RLCU_OK;
}

}  // extern "C"
