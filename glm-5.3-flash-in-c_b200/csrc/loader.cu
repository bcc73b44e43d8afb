// loader.cu - a checkpoint directory streamed straight into the engine's HBM layout.
//
// Replaces, for this engine, the reference's load path: the safetensors index and reads
// (src/io/glm53f_st.c), the tensor-name binding (src/model/glm53f_bind.c:139-206,311-331) and the
// expert geometry (src/io/glm53f_load.c:15-99) - there built around an SSD cache that pulls experts
// on demand, here a one-time stream of every tensor this rank owns into its final place:
//
//   * every *.safetensors file of the directory is indexed from its header (8-byte length, JSON);
//   * each matrix gets its place reserved in the engine (g5b_engine_reserve: same name, shape and
//     dtype checks as g5b_engine_load; routed experts land in the rank's expert slab, experts of
//     other ranks are skipped without being read) and is cut into pieces of at most 32 MB;
//   * reader threads pread the pieces into pinned staging buffers (two per thread) and copy them to
//     the device on a stream of their own, so file reads, PCIe copies and the next read overlap;
//   * vectors (norm weights, biases, conv kernels: BF16 or F32, widened by the engine) are small and
//     go through g5b_engine_load.
// No tensor is ever held whole in host memory; the host footprint is threads x 64 MB of pinned memory.
#include <dirent.h>
#include <fcntl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "kernels.h"

extern "C" int g5b_engine_reserve(g5b_engine *e, const char *name, int dtype, int rows, int cols, void **data_dev,
                                  float **scale_dev);
extern "C" int g5b_engine_wants_vector(g5b_engine *e, const char *name);
extern "C" int g5b_engine_device(const g5b_engine *e);
extern "C" int g5b_engine_layers(const g5b_engine *e);

namespace {

struct StTensor {
    int file = -1;
    int dtype = -1;                  // G5B_DT_*
    std::vector<long> shape;
    size_t begin = 0, end = 0;       // byte range in the file, header included
};

constexpr size_t PIECE = (size_t)32 << 20;
const char *PREFIX = "model.language_model.";

int fail_msg(const char *fmt, const char *a = "", const char *b = "")
{
    char msg[480];
    snprintf(msg, sizeof msg, fmt, a, b);
    g5b::set_last_error(msg);
    fprintf(stderr, "glm53f_b200: %s\n", msg);
    return -1;
}

// The header is one flat JSON object: "name": {"dtype": "...", "shape": [..], "data_offsets": [a, b]}.
// A scanner for exactly that shape: strings (with escapes), integers, nesting one level deep.
struct Scanner {
    const char *p, *end;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\r' || *p == '\t')) p++; }
    bool eat(char c) { ws(); if (p < end && *p == c) { p++; return true; } return false; }
    bool str(std::string &out)
    {
        ws();
        if (p >= end || *p != '"') return false;
        out.clear();
        for (p++; p < end && *p != '"'; p++) {
            if (*p == '\\' && p + 1 < end) { p++; out.push_back(*p); }
            else out.push_back(*p);
        }
        if (p >= end) return false;
        p++;
        return true;
    }
    bool num(long &v)
    {
        ws();
        char *q = nullptr;
        v = strtol(p, &q, 10);
        if (q == p) return false;
        p = q;
        return true;
    }
    // skip any value (used for __metadata__)
    bool skip()
    {
        ws();
        if (p >= end) return false;
        if (*p == '"') { std::string s; return str(s); }
        if (*p == '{' || *p == '[') {
            const char open = *p, close = open == '{' ? '}' : ']';
            p++;
            for (;;) {
                ws();
                if (p >= end) return false;
                if (*p == close) { p++; return true; }
                if (*p == ',' || *p == ':') { p++; continue; }
                if (!skip()) return false;
            }
        }
        while (p < end && *p != ',' && *p != '}' && *p != ']') p++;
        return true;
    }
};

bool parse_header(const std::string &h, size_t data0, int file, std::unordered_map<std::string, StTensor> &out)
{
    Scanner s{h.data(), h.data() + h.size()};
    if (!s.eat('{')) return false;
    while (!s.eat('}')) {
        std::string name;
        if (!s.str(name) || !s.eat(':')) return false;
        if (name == "__metadata__") { if (!s.skip()) return false; s.eat(','); continue; }
        StTensor t;
        t.file = file;
        if (!s.eat('{')) return false;
        while (!s.eat('}')) {
            std::string key;
            if (!s.str(key) || !s.eat(':')) return false;
            if (key == "dtype") {
                std::string d;
                if (!s.str(d)) return false;
                t.dtype = d == "F32" ? G5B_DT_F32 : d == "BF16" ? G5B_DT_BF16 : d == "F8_E4M3" ? G5B_DT_FP8 : -1;
            } else if (key == "shape") {
                if (!s.eat('[')) return false;
                while (!s.eat(']')) { long v; if (!s.num(v)) return false; t.shape.push_back(v); s.eat(','); }
            } else if (key == "data_offsets") {
                long a, b;
                if (!s.eat('[') || !s.num(a) || !s.eat(',') || !s.num(b) || !s.eat(']')) return false;
                t.begin = data0 + (size_t)a; t.end = data0 + (size_t)b;
            } else if (!s.skip()) return false;
            s.eat(',');
        }
        out[name] = t;
        s.eat(',');
    }
    return true;
}

struct Piece { int file; size_t off, bytes; uint8_t *dst; };

}  // namespace

extern "C" int g5b_engine_load_checkpoint(g5b_engine *e, const char *directory, int threads)
{
    if (!e || !directory) return fail_msg("load_checkpoint: null argument");
    if (threads < 1) threads = 4;
    if (threads > 32) threads = 32;
    // ---- index every shard
    std::vector<std::string> files;
    if (DIR *d = opendir(directory)) {
        while (dirent *ent = readdir(d)) {
            const std::string fn = ent->d_name;
            if (fn.size() > 12 && fn.compare(fn.size() - 12, 12, ".safetensors") == 0) files.push_back(std::string(directory) + "/" + fn);
        }
        closedir(d);
    } else return fail_msg("cannot open checkpoint directory %s", directory);
    if (files.empty()) return fail_msg("no .safetensors file in %s", directory);
    std::sort(files.begin(), files.end());
    std::vector<int> fds;
    struct Closer { std::vector<int> &v; ~Closer() { for (int fd : v) if (fd >= 0) close(fd); } } closer{fds};
    std::unordered_map<std::string, StTensor> index;
    for (size_t i = 0; i < files.size(); i++) {
        const int fd = open(files[i].c_str(), O_RDONLY);
        if (fd < 0) return fail_msg("cannot open %s", files[i].c_str());
        fds.push_back(fd);
        uint64_t hlen = 0;
        if (pread(fd, &hlen, 8, 0) != 8 || hlen == 0 || hlen > ((uint64_t)1 << 30)) return fail_msg("%s: bad safetensors header length", files[i].c_str());
        std::string header((size_t)hlen, '\0');
        if (pread(fd, &header[0], (size_t)hlen, 8) != (ssize_t)hlen) return fail_msg("%s: short read of the header", files[i].c_str());
        if (!parse_header(header, 8 + (size_t)hlen, (int)i, index)) return fail_msg("%s: header is not the flat JSON object safetensors writes", files[i].c_str());
    }
    // ---- reserve places, cut matrices into pieces, load vectors directly
    std::vector<Piece> pieces;
    size_t total = 0;
    for (auto &kv : index) {
        const std::string &full = kv.first;
        const StTensor &t = kv.second;
        if (full.size() > 10 && full.compare(full.size() - 10, 10, "_scale_inv") == 0) continue;
        std::string name;
        if (full.compare(0, strlen(PREFIX), PREFIX) == 0) name = full.substr(strlen(PREFIX));
        else if (full == "lm_head.weight") name = full;
        else continue;                                                   // not a tensor of the language model
        if (t.dtype < 0) return fail_msg("%s has a dtype that is not part of this architecture", full.c_str());
        long n = 1;
        for (long v : t.shape) n *= v;
        const size_t eb = t.dtype == G5B_DT_F32 ? 4 : t.dtype == G5B_DT_BF16 ? 2 : 1;
        if (t.end - t.begin != (size_t)n * eb) return fail_msg("%s: byte range does not match its shape", full.c_str());
        // conv kernels are [n][1][k]; every other matrix is 2-D; vectors are 1-D
        const bool is_vector = g5b_engine_wants_vector(e, name.c_str()) != 0;
        if (is_vector) {
            std::vector<uint8_t> buf((size_t)n * eb);
            if (pread(fds[t.file], buf.data(), buf.size(), (off_t)t.begin) != (ssize_t)buf.size()) return fail_msg("%s: short read", full.c_str());
            g5b_tensor gt{buf.data(), nullptr, t.dtype, (int32_t)n, 1, 0};
            if (g5b_engine_load(e, name.c_str(), &gt)) return -1;
            continue;
        }
        if (t.shape.size() != 2) continue;                               // nothing of this engine's (e.g. the MTP layer's extras)
        void *data_dev = nullptr;
        float *scale_dev = nullptr;
        {
            int l = -1;
            if (sscanf(name.c_str(), "layers.%d.", &l) == 1 && l >= g5b_engine_layers(e)) continue;   // a layer beyond this engine's cut
        }
        if (g5b_engine_reserve(e, name.c_str(), t.dtype, (int)t.shape[0], (int)t.shape[1], &data_dev, &scale_dev)) return -1;
        if (!data_dev) continue;                                         // another rank's expert
        for (size_t off = 0; off < t.end - t.begin; off += PIECE)
            pieces.push_back(Piece{t.file, t.begin + off, std::min(PIECE, t.end - t.begin - off), static_cast<uint8_t *>(data_dev) + off});
        total += t.end - t.begin;
        if (t.dtype == G5B_DT_FP8) {
            auto it = index.find(full + "_scale_inv");
            if (it == index.end() || it->second.dtype != G5B_DT_F32) return fail_msg("%s is FP8 but has no F32 %s_scale_inv", full.c_str(), full.c_str());
            const StTensor &sc = it->second;
            pieces.push_back(Piece{sc.file, sc.begin, sc.end - sc.begin, reinterpret_cast<uint8_t *>(scale_dev)});
            total += sc.end - sc.begin;
        }
    }
    // largest first: the tail of the stream is then made of small pieces
    std::sort(pieces.begin(), pieces.end(), [](const Piece &a, const Piece &b) { return a.bytes > b.bytes; });
    // ---- stream
    const int device = g5b_engine_device(e);
    std::atomic<size_t> next{0};
    std::atomic<int> failed{0};
    auto worker = [&]() {
        if (cudaSetDevice(device) != cudaSuccess) { failed = 1; return; }
        cudaStream_t st = nullptr;
        uint8_t *slot[2] = {nullptr, nullptr};
        cudaEvent_t done[2] = {nullptr, nullptr};
        bool ok = cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) == cudaSuccess;
        for (int i = 0; i < 2 && ok; i++)
            ok = cudaHostAlloc((void **)&slot[i], PIECE, cudaHostAllocDefault) == cudaSuccess && cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming) == cudaSuccess;
        for (size_t k = 0, i; ok && !failed && (i = next.fetch_add(1)) < pieces.size(); k++) {
            const Piece &p = pieces[i];
            const int s = (int)(k & 1);
            if (k >= 2) ok = cudaEventSynchronize(done[s]) == cudaSuccess;      // the slot's previous copy has left it
            for (size_t got = 0; ok && got < p.bytes;) {
                const ssize_t r = pread(fds[p.file], slot[s] + got, p.bytes - got, (off_t)(p.off + got));
                if (r <= 0) ok = false; else got += (size_t)r;
            }
            if (ok) ok = cudaMemcpyAsync(p.dst, slot[s], p.bytes, cudaMemcpyHostToDevice, st) == cudaSuccess &&
                         cudaEventRecord(done[s], st) == cudaSuccess;
        }
        if (st) cudaStreamSynchronize(st);
        if (!ok) failed = 1;
        for (int i = 0; i < 2; i++) { if (slot[i]) cudaFreeHost(slot[i]); if (done[i]) cudaEventDestroy(done[i]); }
        if (st) cudaStreamDestroy(st);
    };
    std::vector<std::thread> pool;
    for (int i = 0; i < threads; i++) pool.emplace_back(worker);
    for (auto &t : pool) t.join();
    if (failed) return fail_msg("streaming the checkpoint failed (a read came up short or a copy was refused)");
    return 0;
}
