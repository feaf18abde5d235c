// A miniature of tract's plan loop for one attention layer, in C++, over tract_b200/host/ops.hpp.
// It drives the ops in the order core::plan does for a stateful node — state(), [resolve_symbols, eval]*,
// freeze, more evals, unfreeze + the same evals again, save_to — the way the reference's own tests drive
// InPlaceKvSdpa (transformers/src/ops/inplace_kv_cache.rs:595-658, resume test :898-942).
//
//   plan_driver <in.bin> <out.bin>
// in.bin : int32 {format, dtype, Hq, Hkv, D, n_steps, freeze_at}, int32 S[n_steps], then per step raw
//          q [Hq, S, D], k [Hkv, S, D], v [Hkv, S, D] in `dtype`.
// out.bin: per step the fused op's output [Hq, S, D]; then the outputs of the steps after freeze_at run a
//          second time from the unfrozen state; then int64 past length; then save_to's K and V [Hkv, T, D];
//          then the output of a lone DynKeyValueCache fed with all K inputs (the whole cache, [Hkv, T, D]);
//          then the output of a lone Sdpa over (q of the last step, saved K, saved V).
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <memory>
#include <vector>

#include "../../tract_b200/host/ops.hpp"

using namespace tract_b200;

#define CU(x)                                                                      \
    do {                                                                           \
        cudaError_t e = (x);                                                       \
        if (e != cudaSuccess) {                                                    \
            std::fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e));           \
            std::exit(2);                                                          \
        }                                                                          \
    } while (0)

static std::vector<char> read_all(const char* path) {
    FILE* f = std::fopen(path, "rb");
    if (!f) std::exit(3);
    std::fseek(f, 0, SEEK_END);
    long n = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    std::vector<char> buf(n);
    if (std::fread(buf.data(), 1, n, f) != (size_t)n) std::exit(3);
    std::fclose(f);
    return buf;
}

int main(int argc, char** argv) {
    if (argc != 3) return 1;
    std::vector<char> in = read_all(argv[1]);
    const int32_t* hdr = (const int32_t*)in.data();
    const int format = hdr[0], Hq = hdr[2], Hkv = hdr[3], D = hdr[4], n_steps = hdr[5], freeze_at = hdr[6];
    const DatumType dt = (DatumType)hdr[1];
    const int32_t* S = hdr + 7;
    const char* payload = (const char*)(S + n_steps);
    const int es = size_of(dt);
    int64_t T = 0;
    for (int i = 0; i < n_steps; i++) T += S[i];

    cudaStream_t stream;
    CU(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));  // tract-cuda: one non-blocking stream per thread
    FILE* out = std::fopen(argv[2], "wb");
    try {
        PagedKvSdpa op;
        op.spec = CacheSpec{"kv_cache_0", 2, format, Hkv, D, T + 64, false};
        op.is_causal = true;
        std::unique_ptr<KvState> st(op.state(0));
        DynKeyValueCache lone;
        lone.spec = op.spec;
        lone.spec.name = "k_cache_alone";
        std::unique_ptr<KvState> lone_st(lone.state(0));

        std::vector<const char*> step_ptr(n_steps);
        const char* cur = payload;
        for (int i = 0; i < n_steps; i++) {
            step_ptr[i] = cur;
            cur += (size_t)(Hq + 2 * Hkv) * S[i] * D * es;
        }
        void *dq, *dk, *dv, *dout, *dsave_k, *dsave_v, *dlone;
        const size_t maxS = 512;
        CU(cudaMalloc(&dq, Hq * maxS * D * es));
        CU(cudaMalloc(&dout, Hq * maxS * D * es));
        CU(cudaMalloc(&dk, Hkv * maxS * D * es));
        CU(cudaMalloc(&dv, Hkv * maxS * D * es));
        CU(cudaMalloc(&dsave_k, Hkv * T * D * es));
        CU(cudaMalloc(&dsave_v, Hkv * T * D * es));
        CU(cudaMalloc(&dlone, Hkv * T * D * es));
        std::vector<char> host(Hq * maxS * D * es);
        int64_t expect_len = 0;

        auto run_step = [&](int i, bool feed_lone) {
            const size_t qb = (size_t)Hq * S[i] * D * es, kb = (size_t)Hkv * S[i] * D * es;
            CU(cudaMemcpyAsync(dq, step_ptr[i], qb, cudaMemcpyHostToDevice, stream));
            CU(cudaMemcpyAsync(dk, step_ptr[i] + qb, kb, cudaMemcpyHostToDevice, stream));
            CU(cudaMemcpyAsync(dv, step_ptr[i] + qb + kb, kb, cudaMemcpyHostToDevice, stream));
            DeviceTensor q = DeviceTensor::contiguous(dq, dt, 1, Hq, S[i], D), k = DeviceTensor::contiguous(dk, dt, 1, Hkv, S[i], D),
                         v = DeviceTensor::contiguous(dv, dt, 1, Hkv, S[i], D), o = DeviceTensor::contiguous(dout, dt, 1, Hq, S[i], D);
            if (st->past_len() != expect_len) throw Error("resolve_symbols would bind the wrong past length");
            op.eval(*st, q, k, v, o, stream);
            expect_len += S[i];
            if (feed_lone) DynKeyValueCache::eval(*lone_st, k, dlone, stream);
            CU(cudaMemcpyAsync(host.data(), dout, qb, cudaMemcpyDeviceToHost, stream));
            CU(cudaStreamSynchronize(stream));  // DeviceSync::ToHost
            std::fwrite(host.data(), 1, qb, out);
        };
        int32_t frozen = -1;
        for (int i = 0; i < n_steps; i++) {
            if (i == freeze_at) frozen = st->freeze(stream);
            run_step(i, true);
        }
        const int64_t len_after = st->past_len();
        // resume: back to the frozen state, the same steps again must give the same bytes
        st->unfreeze(frozen);
        expect_len = 0;
        for (int i = 0; i < freeze_at; i++) expect_len += S[i];
        for (int i = freeze_at; i < n_steps; i++) run_step(i, false);
        if (st->past_len() != len_after) throw Error("length after resume differs");
        std::fwrite(&len_after, 8, 1, out);
        st->save_to(dsave_k, dsave_v, dt, stream);
        st->check(stream);
        std::vector<char> big(Hkv * T * D * es);
        for (void* p : {dsave_k, dsave_v, dlone}) {
            CU(cudaMemcpy(big.data(), p, big.size(), cudaMemcpyDeviceToHost));
            std::fwrite(big.data(), 1, big.size(), out);
        }
        // a lone Sdpa node over the saved tensors
        Sdpa sdpa;
        sdpa.is_causal = true, sdpa.datum_type = dt;
        const int last = n_steps - 1;
        CU(cudaMemcpy(dq, step_ptr[last], (size_t)Hq * S[last] * D * es, cudaMemcpyHostToDevice));
        sdpa.eval(DeviceTensor::contiguous(dq, dt, 1, Hq, S[last], D), DeviceTensor::contiguous(dsave_k, dt, 1, Hkv, T, D),
                  DeviceTensor::contiguous(dsave_v, dt, 1, Hkv, T, D), nullptr, DeviceTensor::contiguous(dout, dt, 1, Hq, S[last], D), stream);
        CU(cudaStreamSynchronize(stream));
        CU(cudaMemcpy(host.data(), dout, (size_t)Hq * S[last] * D * es, cudaMemcpyDeviceToHost));
        std::fwrite(host.data(), 1, (size_t)Hq * S[last] * D * es, out);
        // error behaviour: a second load_from on an initialised cache is refused, like every misuse, by exception
        bool threw = false;
        try {
            st->load_from(DeviceTensor::contiguous(dk, dt, 1, Hkv, 1, D), nullptr, stream);
        } catch (const Error&) {
            threw = true;
        }
        if (!threw) throw Error("load_from on an initialised cache must fail");
    } catch (const Error& e) {
        std::fprintf(stderr, "plan_driver: %s\n", e.what());
        return 4;
    }
    std::fclose(out);
    return 0;
}
