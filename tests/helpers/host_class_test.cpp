// Drives include/LatticeFilterKernel.hpp on a GPU: reads a problem from a binary file, runs the op
// both ways (whole batch, and the reference's per-item ComputeKernel + LatticeFilter structure) and
// writes both outputs back.  File layout (little endian): int32 header
// {batch, n_sdims, sdims[3], C, R, bilateral, reverse}, float32 {theta_alpha, theta_beta, theta_gamma},
// then input [batch, n, C] and reference [batch, n, R] as float32, or as float64 when the program is
// given "f64" as its third argument (the outputs then are float64 too).
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "LatticeFilterKernel.hpp"

static void die(const char* what) {
    fprintf(stderr, "host_class_test: %s\n", what);
    exit(2);
}

template <typename T>
static int run(FILE* f, const char* out_path) {
    int hdr[9];
    float theta[3];
    if (fread(hdr, 4, 9, f) != 9 || fread(theta, 4, 3, f) != 3) die("short header");
    const int batch = hdr[0], n_sdims = hdr[1], C = hdr[5], R = hdr[6], bilateral = hdr[7], reverse = hdr[8];
    std::vector<int> shape = {batch};
    size_t n = 1;
    for (int i = 0; i < n_sdims; i++) { shape.push_back(hdr[2 + i]); n *= hdr[2 + i]; }
    shape.push_back(C);
    std::vector<T> in(batch * n * C), ref(batch * n * R), out(batch * n * C), out2(batch * n * C);
    if (fread(in.data(), sizeof(T), in.size(), f) != in.size()) die("short input");
    if (R && fread(ref.data(), sizeof(T), ref.size(), f) != ref.size()) die("short reference");
    fclose(f);

    T *d_in, *d_ref = nullptr, *d_out, *d_pos;
    cudaStream_t stream;
    if (cudaStreamCreate(&stream) != cudaSuccess) die("no CUDA device");
    cudaMalloc(&d_in, in.size() * sizeof(T));
    cudaMalloc(&d_out, out.size() * sizeof(T));
    if (R) cudaMalloc(&d_ref, ref.size() * sizeof(T));
    cudaMalloc(&d_pos, n * (n_sdims + R) * sizeof(T) + 16);
    cudaMemcpyAsync(d_in, in.data(), in.size() * sizeof(T), cudaMemcpyHostToDevice, stream);
    if (R) cudaMemcpyAsync(d_ref, ref.data(), ref.size() * sizeof(T), cudaMemcpyHostToDevice, stream);

    int n_allocs = 0;
    long long sized_entries = 0, sized_bound = 0;
    pl::OpContext context([&](size_t bytes) { void* p = nullptr; cudaMalloc(&p, bytes); n_allocs++; return p; },
                          [](void* p) { cudaFree(p); });
    pl::GpuDevice device{stream};
    try {
        pl::LatticeFilterOpT<T> op(reverse != 0, bilateral != 0, theta[0], theta[1], theta[2]);
        op.Compute(device, &context, d_in, shape, d_ref, R, d_out);
        cudaMemcpyAsync(out.data(), d_out, out.size() * sizeof(T), cudaMemcpyDeviceToHost, stream);
        op.ComputePerItem(device, &context, d_in, shape, d_ref, R, d_pos, d_out);
        cudaMemcpyAsync(out2.data(), d_out, out2.size() * sizeof(T), cudaMemcpyDeviceToHost, stream);
        // the same op with a workspace sized from a (far too small) entry bound: verified and repeated until it fits
        {
            std::vector<T> out3(out.size());
            const pl_stats st = op.ComputeSized(device, &context, d_in, shape, d_ref, R, d_out, 64);
            cudaMemcpyAsync(out3.data(), d_out, out3.size() * sizeof(T), cudaMemcpyDeviceToHost, stream);
            if (cudaStreamSynchronize(stream) != cudaSuccess) die("stream failed");
            if (st.device_status != PL_OK || st.num_entries <= 64 || st.max_entries < st.num_entries)
                die("ComputeSized: unexpected counters");
            double worst = 0;
            for (size_t i = 0; i < out.size(); i++) {
                const double diff = (double)out3[i] - (double)out[i];
                if (!(diff == diff)) die("ComputeSized: NaN in the output");
                if (diff < 0 ? -diff > worst : diff > worst) worst = diff < 0 ? -diff : diff;
            }
            if (worst > 1e-4) die("ComputeSized: output differs from Compute");
            sized_entries = (long long)st.num_entries;
            sized_bound = (long long)st.max_entries;
        }
        // an unsupported position dimension must surface as an exception, not abort the process
        bool threw = false;
        try {
            pl::LatticeFilter<pl::GpuDevice, T>()(device, &context, d_out, d_in, d_pos, 16, 11, 4, false);
        } catch (const pl::Error& e) {
            threw = e.status == PL_UNSUPPORTED_DIMS;
        }
        if (!threw) die("unsupported dims did not throw");
    } catch (const pl::Error& e) {
        fprintf(stderr, "host_class_test: %s\n", e.what());
        return 3;
    }
    if (cudaStreamSynchronize(stream) != cudaSuccess) die("stream failed");
    f = fopen(out_path, "wb");
    fwrite(out.data(), sizeof(T), out.size(), f);
    fwrite(out2.data(), sizeof(T), out2.size(), f);
    fclose(f);
    printf("ok allocs=%d sized_entries=%lld sized_bound=%lld\n", n_allocs, sized_entries, sized_bound);
    return 0;
}

int main(int argc, char** argv) {
    if (argc != 3 && argc != 4) die("usage: host_class_test <in> <out> [f64]");
    FILE* f = fopen(argv[1], "rb");
    if (!f) die("cannot open input");
    if (argc == 4 && strcmp(argv[3], "f64") == 0) return run<double>(f, argv[2]);
    return run<float>(f, argv[2]);
}
