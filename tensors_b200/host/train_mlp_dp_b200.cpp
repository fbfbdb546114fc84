// Data-parallel MLP training over libtfb's C-ABI from plain C++ (no CUDA headers, no Python): the
// reference example's loop (examples/train_mlp.cpp:161-183: forward, loss, backward, update) for the
// layer sizes of the data-parallel configuration, with the documented momentum update
// (nn/optim/SGD.hpp:3-6), run as R ranks inside ONE process.
//
//   train_mlp_dp_b200 <problem file> <ranks> <steps> <output file> [lr] [momentum]
//
// Ranks map to GPUs round-robin. With one visible GPU all ranks live on it and their gradient
// exchange runs as one cooperative launch (tfb_mlp_exchange_update_one_device); with at least R GPUs
// every rank gets its own device and a host thread, the handles are connected with
// tfb_mlp_connect_local, and each rank's step ends in the fused peer-memory exchange kernel.
//
// Problem file (little-endian): int64 L, int64 dims[L+1], int64 batch, then for each layer the weight
// [out,in] and the bias [out] as float32, then X [batch, dims[0]] float32 and labels [batch] int64.
// Output file: float32 loss of the LAST step, int64 numel, float32 params[numel] of rank 0 after the
// last step, float32 summed gradient[numel] of the last step (assembled from the ranks' slices), and
// one int64 per rank: 1 if that rank's parameters are bit-identical to rank 0's.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "../../include/tfb.h"

namespace {

void ok(int rc, const char* what) {
    if (rc != TFB_OK) throw std::runtime_error(std::string(what) + ": " + tfb_last_error_string());
}

template <typename T>
void read_exact(std::FILE* f, T* dst, size_t n) {
    if (n != 0 && std::fread(dst, sizeof(T), n, f) != n) throw std::runtime_error("problem file is truncated");
}

struct Rank {
    int device = 0;
    tfb_mlp* mlp = nullptr;
    void* stream = nullptr;
    float* X = nullptr;
    int64_t* labels = nullptr;
    int64_t row0 = 0, rows = 0;
};

void* device_ptr(tfb_mlp* m, int which) {
    void* p = nullptr;
    ok(tfb_mlp_buffer(m, which, 0, &p), "tfb_mlp_buffer");
    return p;
}

}  // namespace

int main(int argc, char** argv) {
    if (argc < 5) {
        std::fprintf(stderr, "usage: %s <problem file> <ranks> <steps> <output file> [lr] [momentum]\n", argv[0]);
        return 64;
    }
    const int world = std::atoi(argv[2]), steps = std::atoi(argv[3]);
    const float lr = argc > 5 ? std::strtof(argv[5], nullptr) : 0.1f;
    const float mu = argc > 6 ? std::strtof(argv[6], nullptr) : 0.9f;
    try {
        if (world < 1 || world > 8 || steps < 1) throw std::runtime_error("1..8 ranks, at least one step");
        std::FILE* f = std::fopen(argv[1], "rb");
        if (f == nullptr) throw std::runtime_error("cannot open the problem file");
        int64_t L = 0;
        read_exact(f, &L, 1);
        if (L < 1 || L > 64) throw std::runtime_error("bad layer count");
        std::vector<int64_t> dims(static_cast<size_t>(L) + 1);
        read_exact(f, dims.data(), dims.size());
        int64_t batch = 0;
        read_exact(f, &batch, 1);
        std::vector<std::vector<float>> W(static_cast<size_t>(L)), B(static_cast<size_t>(L));
        for (int64_t i = 0; i < L; ++i) {
            W[i].resize(static_cast<size_t>(dims[i + 1] * dims[i]));
            B[i].resize(static_cast<size_t>(dims[i + 1]));
            read_exact(f, W[i].data(), W[i].size());
            read_exact(f, B[i].data(), B[i].size());
        }
        std::vector<float> X(static_cast<size_t>(batch * dims[0]));
        std::vector<int64_t> labels(static_cast<size_t>(batch));
        read_exact(f, X.data(), X.size());
        read_exact(f, labels.data(), labels.size());
        std::fclose(f);

        int visible = 0;
        ok(tfb_device_count(&visible), "tfb_device_count");
        if (visible < 1) throw std::runtime_error("no CUDA device");
        const bool one_device = visible < world;
        std::vector<Rank> ranks(static_cast<size_t>(world));
        const int64_t base = batch / world, extra = batch % world;
        for (int r = 0; r < world; ++r) {
            Rank& k = ranks[r];
            k.device = one_device ? 0 : r;
            k.row0 = r * base + (r < extra ? r : extra);
            k.rows = base + (r < extra ? 1 : 0);
            ok(tfb_set_device(k.device), "tfb_set_device");
            ok(tfb_stream_create(k.device, &k.stream), "tfb_stream_create");
            ok(tfb_mlp_create(static_cast<int>(L), dims.data(), k.rows > 0 ? k.rows : 1, &k.mlp), "tfb_mlp_create");
            float* params = static_cast<float*>(device_ptr(k.mlp, TFB_MLP_PARAMS));
            for (int64_t i = 0; i < L; ++i) {
                int64_t wo = 0, bo = 0;
                ok(tfb_mlp_segment(k.mlp, static_cast<int>(i), &wo, &bo), "tfb_mlp_segment");
                ok(tfb_memcpy(params + wo, W[i].data(), W[i].size() * 4, 1, k.stream), "tfb_memcpy");
                ok(tfb_memcpy(params + bo, B[i].data(), B[i].size() * 4, 1, k.stream), "tfb_memcpy");
            }
            void* p = nullptr;
            ok(tfb_alloc(k.device, static_cast<size_t>(k.rows * dims[0]) * 4, k.stream, &p), "tfb_alloc");
            k.X = static_cast<float*>(p);
            ok(tfb_alloc(k.device, static_cast<size_t>(k.rows) * 8, k.stream, &p), "tfb_alloc");
            k.labels = static_cast<int64_t*>(p);
            ok(tfb_memcpy(k.X, X.data() + k.row0 * dims[0], static_cast<size_t>(k.rows * dims[0]) * 4, 1, k.stream),
               "tfb_memcpy");
            ok(tfb_memcpy(k.labels, labels.data() + k.row0, static_cast<size_t>(k.rows) * 8, 1, k.stream), "tfb_memcpy");
            ok(tfb_mlp_set_option(k.mlp, TFB_MLP_OPT_KEEP_REDUCED_GRADS, 1), "tfb_mlp_set_option");
            ok(tfb_stream_synchronize(k.stream), "tfb_stream_synchronize");
        }
        std::vector<tfb_mlp*> handles;
        for (Rank& k : ranks) handles.push_back(k.mlp);
        if (one_device) {
            std::vector<void*> regions;
            for (Rank& k : ranks) regions.push_back(device_ptr(k.mlp, TFB_MLP_REGION));
            for (int r = 0; r < world; ++r) ok(tfb_mlp_connect_ptrs(ranks[r].mlp, r, world, regions.data()), "tfb_mlp_connect_ptrs");
        } else {
            ok(tfb_mlp_connect_local(handles.data(), world), "tfb_mlp_connect_local");
        }

        if (one_device) {
            // all ranks on one stream of one device: their steps run one after the other, the exchange
            // of all of them as one cooperative launch
            void* stream = ranks[0].stream;
            for (int s = 0; s < steps; ++s) {
                for (Rank& k : ranks)
                    ok(tfb_mlp_forward_backward(k.mlp, k.X, k.labels, k.rows, batch, stream), "tfb_mlp_forward_backward");
                ok(tfb_mlp_exchange_update_one_device(handles.data(), world, lr, mu, stream),
                   "tfb_mlp_exchange_update_one_device");
            }
            ok(tfb_stream_synchronize(stream), "tfb_stream_synchronize");
        } else {
            // one host thread per rank, each with its own device current; the ranks meet inside the
            // exchange kernel, not on the host
            std::vector<std::string> errors(static_cast<size_t>(world));
            std::vector<std::thread> threads;
            for (int r = 0; r < world; ++r)
                threads.emplace_back([&, r] {
                    try {
                        Rank& k = ranks[r];
                        ok(tfb_set_device(k.device), "tfb_set_device");
                        for (int s = 0; s < steps; ++s)
                            ok(tfb_mlp_step(k.mlp, k.X, k.labels, k.rows, batch, lr, mu, k.stream), "tfb_mlp_step");
                        ok(tfb_stream_synchronize(k.stream), "tfb_stream_synchronize");
                    } catch (const std::exception& e) {
                        errors[r] = e.what();
                    }
                });
            for (std::thread& t : threads) t.join();
            for (const std::string& e : errors)
                if (!e.empty()) throw std::runtime_error(e);
        }

        // results
        const int64_t numel = tfb_mlp_numel(ranks[0].mlp);
        std::vector<float> params0(static_cast<size_t>(numel)), grads(static_cast<size_t>(numel), 0.f);
        std::vector<int64_t> same(static_cast<size_t>(world), 0);
        float loss = 0.f;
        for (int r = 0; r < world; ++r) {
            Rank& k = ranks[r];
            ok(tfb_set_device(k.device), "tfb_set_device");
            int code = 0;
            if (tfb_device_status(&code) != TFB_OK || code != 0)
                throw std::runtime_error("device error " + std::to_string(code) + " on rank " + std::to_string(r));
            std::vector<float> p(static_cast<size_t>(numel));
            ok(tfb_memcpy(p.data(), device_ptr(k.mlp, TFB_MLP_PARAMS), static_cast<size_t>(numel) * 4, 2, k.stream), "tfb_memcpy");
            // this rank's slice of the summed gradient (whole vectors of four floats, like the kernel)
            const int64_t n_vec = numel / 4, lo = 4 * (n_vec * r / world), hi = 4 * (n_vec * (r + 1) / world);
            ok(tfb_memcpy(grads.data() + lo, static_cast<float*>(device_ptr(k.mlp, TFB_MLP_REDUCED_GRADS)) + lo,
                          static_cast<size_t>(hi - lo) * 4, 2, k.stream), "tfb_memcpy");
            if (r == 0) ok(tfb_memcpy(&loss, device_ptr(k.mlp, TFB_MLP_LOSS), 4, 2, k.stream), "tfb_memcpy");
            ok(tfb_stream_synchronize(k.stream), "tfb_stream_synchronize");
            if (r == 0) params0 = p;
            same[r] = std::memcmp(p.data(), params0.data(), static_cast<size_t>(numel) * 4) == 0 ? 1 : 0;
        }
        std::FILE* o = std::fopen(argv[4], "wb");
        if (o == nullptr) throw std::runtime_error("cannot open the output file");
        std::fwrite(&loss, 4, 1, o);
        std::fwrite(&numel, 8, 1, o);
        std::fwrite(params0.data(), 4, params0.size(), o);
        std::fwrite(grads.data(), 4, grads.size(), o);
        std::fwrite(same.data(), 8, same.size(), o);
        std::fclose(o);
        for (Rank& k : ranks) {
            ok(tfb_set_device(k.device), "tfb_set_device");
            ok(tfb_free(k.X, k.device, k.stream), "tfb_free");
            ok(tfb_free(k.labels, k.device, k.stream), "tfb_free");
            ok(tfb_stream_synchronize(k.stream), "tfb_stream_synchronize");
        }
        if (!one_device)   // unmap the peers everywhere before any region is released
            for (Rank& k : ranks) {
                ok(tfb_set_device(k.device), "tfb_set_device");
                ok(tfb_mlp_connect_ptrs(k.mlp, 0, 1, nullptr), "tfb_mlp_connect_ptrs");
            }
        for (Rank& k : ranks) {
            ok(tfb_set_device(k.device), "tfb_set_device");
            ok(tfb_mlp_destroy(k.mlp), "tfb_mlp_destroy");
            ok(tfb_stream_destroy(k.stream), "tfb_stream_destroy");
        }
        std::printf("[train_mlp_dp_b200] ranks=%d devices=%d steps=%d loss=%.6f\n", world, one_device ? 1 : world, steps, loss);
        return 0;
    } catch (const std::exception& e) {
        std::printf("exception: %s\n", e.what());
        return 2;
    }
}
