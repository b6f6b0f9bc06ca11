// C++ host layer over the C ABI (pl_lattice.h): the reference's device functors and op class with
// their own parameter lists, for callers that used src/LatticeFilterKernel.h.
//
//   pl::ComputeKernel<pl::GpuDevice, T>     <->  ComputeKernel<GPUDevice, T>   src/LatticeFilterKernel.h:40-54
//   pl::LatticeFilter<pl::GpuDevice, T>     <->  LatticeFilter<GPUDevice, T>   src/LatticeFilterKernel.h:28-38
//   pl::LatticeFilterOpT<T>                 <->  LatticeFilterOp<GPUDevice, T> src/LatticeFilterKernel.cpp:87-181
//   (pl::LatticeFilterOp = LatticeFilterOpT<float>), for T = float and T = double, the two types the
//   reference instantiates (src/LatticeFilterKernel.cu:105-108).
//
// The TensorFlow slots become two small types: GpuDevice carries the stream (Eigen::GpuDevice::stream()),
// OpContext lends scratch memory the way OpKernelContext::allocate_temp does.  Errors are C++ exceptions
// carrying the pl_status (the reference aborts the process: LOG(FATAL), exit, throw 1).
#ifndef PL_LATTICE_FILTER_KERNEL_HPP
#define PL_LATTICE_FILTER_KERNEL_HPP

#include <cstddef>
#include <cstdint>
#include <functional>
#include <stdexcept>
#include <string>
#include <vector>

#include "pl_lattice.h"

namespace pl {

struct Error : std::runtime_error {
    int status;
    Error(int status_, const std::string& where)
        : std::runtime_error(where + ": " + pl_strerror(status_) +
                             (status_ == PL_CUDA_ERROR ? std::string(" (") + pl_last_cuda_error() + ")" : "")),
          status(status_) {}
};

inline void check(int status, const char* where) {
    if (status != PL_OK) throw Error(status, where);
}

// Stands for Eigen::GpuDevice: the stream all work is ordered on (a cudaStream_t).
struct GpuDevice {
    void* stream_ = nullptr;
    void* stream() const { return stream_; }
};

// Stands for OpKernelContext: lends device scratch for the duration of one Compute.  The caller
// supplies the allocator (a framework's temp allocator, a pool, cudaMalloc...); this layer never
// allocates device memory by itself.  The buffer is kept and reused while it is large enough.
class OpContext {
public:
    using Alloc = std::function<void*(size_t)>;
    using Free = std::function<void(void*)>;
    OpContext(Alloc alloc, Free free) : alloc_(std::move(alloc)), free_(std::move(free)) {}
    ~OpContext() { release(); }
    OpContext(const OpContext&) = delete;
    OpContext& operator=(const OpContext&) = delete;

    void* allocate_temp(size_t bytes) {
        if (bytes > bytes_) {
            release();
            ptr_ = alloc_(bytes);
            if (!ptr_) throw Error(PL_WORKSPACE_TOO_SMALL, "OpContext::allocate_temp");
            bytes_ = bytes;
        }
        return ptr_;
    }
    size_t temp_bytes() const { return bytes_; }
    void* temp() const { return ptr_; }
    void release() {
        if (ptr_) free_(ptr_);
        ptr_ = nullptr;
        bytes_ = 0;
    }

private:
    Alloc alloc_;
    Free free_;
    void* ptr_ = nullptr;
    size_t bytes_ = 0;
};

// The C entry points of each number type.
template <typename T>
struct Abi;
template <>
struct Abi<float> {
    static int workspace_bytes(int batch, int n, int pd, int vd, int nsd, const int* sd, size_t* bytes,
                               int64_t max_entries = 0) {
        return pl_workspace_bytes(batch, n, pd, vd, nsd, sd, max_entries, PL_MODE_ATOMIC, bytes);
    }
    static int compute_positions(const float* ref, float* pos, int n, int r, int nsd, const int* sd, float s_std,
                                 float f_std, void* stream) {
        return pl_compute_positions_f32(ref, pos, n, r, nsd, sd, s_std, f_std, stream);
    }
    static int filter(float* out, const float* in, const float* pos, int batch, int n, int pd, int vd, int reverse,
                      void* ws, size_t ws_bytes, void* stream) {
        return pl_filter_f32(out, in, pos, batch, n, pd, vd, reverse, ws, ws_bytes, 0, PL_MODE_ATOMIC, stream);
    }
    static int lattice_filter(float* out, const float* in, const float* ref, int batch, int nsd, const int* sd,
                              int c, int r, int bilateral, float ta, float tb, float tg, int reverse, void* ws,
                              size_t ws_bytes, void* stream, int64_t max_entries = 0) {
        return pl_lattice_filter_f32(out, in, ref, batch, nsd, sd, c, r, bilateral, ta, tb, tg, reverse, ws,
                                     ws_bytes, max_entries, PL_MODE_ATOMIC, stream);
    }
};
template <>
struct Abi<double> {
    static int workspace_bytes(int batch, int n, int pd, int vd, int nsd, const int* sd, size_t* bytes,
                               int64_t max_entries = 0) {
        return pl_workspace_bytes_f64(batch, n, pd, vd, nsd, sd, max_entries, bytes);
    }
    static int compute_positions(const double* ref, double* pos, int n, int r, int nsd, const int* sd,
                                 double s_std, double f_std, void* stream) {
        return pl_compute_positions_f64(ref, pos, n, r, nsd, sd, s_std, f_std, stream);
    }
    static int filter(double* out, const double* in, const double* pos, int batch, int n, int pd, int vd,
                      int reverse, void* ws, size_t ws_bytes, void* stream) {
        return pl_filter_f64(out, in, pos, batch, n, pd, vd, reverse, ws, ws_bytes, 0, stream);
    }
    static int lattice_filter(double* out, const double* in, const double* ref, int batch, int nsd, const int* sd,
                              int c, int r, int bilateral, double ta, double tb, double tg, int reverse, void* ws,
                              size_t ws_bytes, void* stream, int64_t max_entries = 0) {
        return pl_lattice_filter_f64(out, in, ref, batch, nsd, sd, c, r, bilateral, ta, tb, tg, reverse, ws,
                                     ws_bytes, max_entries, stream);
    }
};

template <typename Device, typename T>
struct ComputeKernel;
template <typename Device, typename T>
struct LatticeFilter;

// positions <- [coordinate / spatial_std ..., reference / features_std ...] for one batch item.
template <typename T>
struct ComputeKernel<GpuDevice, T> {
    void operator()(const GpuDevice& d, OpContext* /*context*/, const T* reference_image, T* positions,
                    int num_super_pixels, int n_spatial_dims, int* spatial_dims /* host */,
                    int n_reference_channels, T spatial_std, T features_std) {
        check(Abi<T>::compute_positions(reference_image, positions, num_super_pixels, n_reference_channels,
                                        n_spatial_dims, spatial_dims, spatial_std, features_std, d.stream()),
              "ComputeKernel");
    }
};

// output <- lattice filter of input at positions, one batch item (any supported pd, vd at run time;
// the reference accepts exactly one compiled pair, src/LatticeFilterKernel.cu:87-100).
template <typename T>
struct LatticeFilter<GpuDevice, T> {
    void operator()(const GpuDevice& d, OpContext* context, T* output, const T* input, const T* positions,
                    int num_super_pixels, int pd, int vd, bool reverse) {
        size_t bytes = 0;
        check(Abi<T>::workspace_bytes(1, num_super_pixels, pd, vd, 0, nullptr, &bytes), "LatticeFilter");
        void* ws = context->allocate_temp(bytes);
        check(Abi<T>::filter(output, input, positions, 1, num_super_pixels, pd, vd, reverse ? 1 : 0, ws,
                             context->temp_bytes(), d.stream()),
              "LatticeFilter");
    }
};

// The op: attributes at construction, Compute on device tensors [batch, *spatial, channels].
template <typename T>
class LatticeFilterOpT {
public:
    LatticeFilterOpT(bool reverse = false, bool bilateral = true, float theta_alpha = 1.f, float theta_beta = 1.f,
                     float theta_gamma = 1.f)
        : reverse_(reverse), bilateral_(bilateral), theta_alpha_(theta_alpha), theta_beta_(theta_beta),
          theta_gamma_(theta_gamma) {}

    // input_shape = {batch, s_1..s_k, channels}; reference has the same batch and spatial dims and
    // n_reference_channels channels (ignored when bilateral is false).  One launch sequence for the
    // whole batch, features fused (no positions tensor).
    void Compute(const GpuDevice& d, OpContext* context, const T* input, const std::vector<int>& input_shape,
                 const T* reference, int n_reference_channels, T* output) const {
        if (input_shape.size() < 3) throw Error(PL_INVALID_ARGUMENT, "LatticeFilterOp::Compute");
        const int batch = input_shape.front(), channels = input_shape.back();
        std::vector<int> sdims(input_shape.begin() + 1, input_shape.end() - 1);
        long long n = 1;
        for (int s : sdims) n *= s;
        const int pd = (int)sdims.size() + (bilateral_ ? n_reference_channels : 0), vd = channels + 1;
        if (batch == 0 || n == 0) return;
        size_t bytes = 0;
        check(Abi<T>::workspace_bytes(batch, (int)n, pd, vd, (int)sdims.size(), sdims.data(), &bytes),
              "LatticeFilterOp::Compute");
        void* ws = context->allocate_temp(bytes);
        // the attributes are floats (src/LatticeFilterKernel.cpp:36-38) and widen to T as in the reference
        check(Abi<T>::lattice_filter(output, input, reference, batch, (int)sdims.size(), sdims.data(), channels,
                                     n_reference_channels, bilateral_ ? 1 : 0, theta_alpha_, theta_beta_,
                                     theta_gamma_, reverse_ ? 1 : 0, ws, context->temp_bytes(), d.stream()),
              "LatticeFilterOp::Compute");
    }

    // Compute with a workspace sized for `max_entries` lattice entries instead of the bound that can never
    // overflow (batch * points * (pd + 1), several times what lattices need).  Whether the lattice fitted is
    // known on the device only: the status is read after the call (this SYNCHRONISES the stream) and the call
    // is repeated with four times the bound as long as it did not fit (a call that did not fit has filled
    // `output` with NaN).  Returns the counters of the call that succeeded: stats.num_entries is what this data
    // needed, a bound for the next call on similar data.  The reference allocates its worst case on every
    // call (src/PermutohedralLatticeGPU.cuh:434-451).
    pl_stats ComputeSized(const GpuDevice& d, OpContext* context, const T* input,
                          const std::vector<int>& input_shape, const T* reference, int n_reference_channels,
                          T* output, int64_t max_entries) const {
        if (input_shape.size() < 3) throw Error(PL_INVALID_ARGUMENT, "LatticeFilterOp::ComputeSized");
        const int batch = input_shape.front(), channels = input_shape.back();
        std::vector<int> sdims(input_shape.begin() + 1, input_shape.end() - 1);
        long long n = 1;
        for (int s : sdims) n *= s;
        const int pd = (int)sdims.size() + (bilateral_ ? n_reference_channels : 0), vd = channels + 1;
        pl_stats stats = {};
        if (batch == 0 || n == 0) return stats;
        const int64_t worst = (int64_t)batch * n * (pd + 1);
        for (;;) {
            if (max_entries <= 0 || max_entries >= worst) max_entries = 0;   // 0: the worst case
            size_t bytes = 0;
            check(Abi<T>::workspace_bytes(batch, (int)n, pd, vd, (int)sdims.size(), sdims.data(), &bytes, max_entries),
                  "LatticeFilterOp::ComputeSized");
            void* ws = context->allocate_temp(bytes);
            check(Abi<T>::lattice_filter(output, input, reference, batch, (int)sdims.size(), sdims.data(), channels,
                                         n_reference_channels, bilateral_ ? 1 : 0, theta_alpha_, theta_beta_,
                                         theta_gamma_, reverse_ ? 1 : 0, ws, context->temp_bytes(), d.stream(),
                                         max_entries),
                  "LatticeFilterOp::ComputeSized");
            check(pl_lattice_stats(ws, &stats, d.stream()), "LatticeFilterOp::ComputeSized");
            if (stats.device_status == PL_CAPACITY_EXCEEDED && max_entries > 0) {
                max_entries *= 4;
                continue;
            }
            if (stats.device_status != PL_OK) throw Error(stats.device_status, "LatticeFilterOp::ComputeSized (device)");
            return stats;
        }
    }

    // The reference's own structure (src/LatticeFilterKernel.cpp:145-179): a positions buffer, then
    // ComputeKernel + LatticeFilter per batch item.  positions must hold n * pd values (device).
    void ComputePerItem(const GpuDevice& d, OpContext* context, const T* input,
                        const std::vector<int>& input_shape, const T* reference, int n_reference_channels,
                        T* positions, T* output) const {
        if (input_shape.size() < 3) throw Error(PL_INVALID_ARGUMENT, "LatticeFilterOp::ComputePerItem");
        const int batch = input_shape.front(), channels = input_shape.back();
        std::vector<int> sdims(input_shape.begin() + 1, input_shape.end() - 1);
        long long n = 1;
        for (int s : sdims) n *= s;
        const int r = bilateral_ ? n_reference_channels : 0;
        const int pd = (int)sdims.size() + r, vd = channels + 1;
        const T spatial_std = bilateral_ ? theta_alpha_ : theta_gamma_;
        const T features_std = bilateral_ ? theta_beta_ : -1.f;
        for (int b = 0; b < batch; b++) {
            ComputeKernel<GpuDevice, T>()(d, context, r ? reference + (size_t)b * n * r : nullptr, positions,
                                          (int)n, (int)sdims.size(), sdims.data(), r, spatial_std, features_std);
            LatticeFilter<GpuDevice, T>()(d, context, output + (size_t)b * n * channels,
                                          input + (size_t)b * n * channels, positions, (int)n, pd, vd, reverse_);
        }
    }

private:
    bool reverse_, bilateral_;
    float theta_alpha_, theta_beta_, theta_gamma_;
};

using LatticeFilterOp = LatticeFilterOpT<float>;

}  // namespace pl
#endif  // PL_LATTICE_FILTER_KERNEL_HPP
