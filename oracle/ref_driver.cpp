// C entry points around the reference's own CPU code for this path - TEST INFRASTRUCTURE, not part of the product.
// Compiles src/cpu_expert.h and src/gguf.h of the reference tree where they lie (include path given by the Makefile);
// nothing of the reference is copied into this repository. The resulting oracle/_ref/libmoex_ref.so validates
// oracle.c, generates the golden vectors under tests/golden/, and is the timed CPU baseline ("reference" kind).
#include <cstring>
#include <cstdio>
#include <memory>
#include <map>
#include "cpu_expert.h"
#include "gguf.h"

static CpuExperts& experts(int threads, bool zp) {
    static std::map<int, std::unique_ptr<CpuExperts>> pool;
    auto& p = pool[threads];
    if (!p) p = std::make_unique<CpuExperts>(threads);
    p->zp = zp;
    return *p;
}

static constexpr size_t QB = (size_t)3 * 2048 * 512 / 2;

static std::vector<CpuExperts::Job> make_jobs(int njobs, const uint8_t* const* blobs, const int* job_start, const int* toks,
                                              const int* pids, const float* ws) {
    std::vector<CpuExperts::Job> jobs;
    for (int j = 0; j < njobs; j++) {
        CpuExperts::Job jb{blobs[j], (const float*)(blobs[j] + QB), {}, {}, {}};
        for (int k = job_start[j]; k < job_start[j + 1]; k++) { jb.toks.push_back(toks[k]); jb.pids.push_back(pids[k]); jb.ws.push_back(ws[k]); }
        jobs.push_back(std::move(jb));
    }
    return jobs;
}

extern "C" {

// CpuExperts::run: the reference's decode path (int8 activations). blobs in the reference layout [nibbles | scale part].
void ref_run(int threads, int zp, int m, const uint8_t* const* blobs, const float* w, const float* x, float* out) {
    std::vector<const uint8_t*> q(m); std::vector<const float*> sc(m);
    for (int j = 0; j < m; j++) { q[j] = blobs[j]; sc[j] = (const float*)(blobs[j] + QB); }
    experts(threads, zp != 0).run(m, q.data(), sc.data(), w, x, out);
}

// CpuExperts::run_pairs: fp32, the parity oracle
void ref_run_pairs(int threads, int zp, int njobs, const uint8_t* const* blobs, const int* job_start, const int* toks,
                   const int* pids, const float* ws, const float* X, int T, int npairs, float* ypair) {
    auto jobs = make_jobs(njobs, blobs, job_start, toks, pids, ws);
    experts(threads, zp != 0).run_pairs(jobs, X, T, npairs, ypair);
}

// CpuExperts::run_pairs_small: int8 activations, at most 9 pairs per job
void ref_run_pairs_small(int threads, int zp, int njobs, const uint8_t* const* blobs, const int* job_start, const int* toks,
                         const int* pids, const float* ws, const float* X, int T, float* ypair) {
    auto jobs = make_jobs(njobs, blobs, job_start, toks, pids, ws);
    experts(threads, zp != 0).run_pairs_small(jobs, X, T, ypair);
}

int ref_gg_dequant(unsigned type, const uint8_t* p, long long n, float* y) {
    try { gg_dequant(type, p, n, y); } catch (const std::exception&) { return -1; }
    return 0;
}
void ref_gg_zp_row(unsigned type, const uint8_t* src, int cols, uint8_t* qb, uint8_t* cs, uint16_t* sup, float* w) {
    gg_zp_row(type, src, cols, qb, cs, sup, w);
}
float ref_gg_zp_at(const uint8_t* qb, const uint8_t* cs, const uint16_t* sup, int i) { return gg_zp_at(qb, cs, sup, i); }
int ref_has_avxvnni() { return cpu_has_avxvnni() ? 1 : 0; }

// The reference's own GGUF reader (struct Gguf, gguf.h:345-462) on a file: for one tensor its dimensions, ggml type,
// the offset of its data from the start of the file and the bytes of one row. Returns the number of dimensions, -1
// when the reader throws (message copied to err), -2 when the tensor is absent. The mapping stays for the process
// lifetime, as in the reference.
int ref_gguf_tensor(const char* path, const char* name, long long* ne, unsigned* type, long long* offset, long long* row_bytes,
                    char* err, int err_len) {
    try {
        Gguf g(path);
        if (!g.has(name)) return -2;
        const Gguf::Tensor& t = g.at(name);
        for (size_t d = 0; d < t.ne.size(); d++) ne[d] = t.ne[d];
        *type = t.type;
        *offset = t.data ? (long long)(t.data - g.base) : -1;
        *row_bytes = t.row_bytes;
        return (int)t.ne.size();
    } catch (const std::exception& e) {
        if (err && err_len > 0) { strncpy(err, e.what(), err_len - 1); err[err_len - 1] = 0; }
        return -1;
    }
}

}
