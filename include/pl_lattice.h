/* C ABI of the B200 permutohedral-lattice filter library (libpl_lattice.so).
 *
 * Plain pointers and sizes only.  Every pointer named "device" is a CUDA device pointer of the
 * current device; everything runs stream-ordered on `stream` (a cudaStream_t passed as void*).
 * Unless a comment says otherwise no call synchronises with the host, allocates, or keeps state
 * between calls: the caller owns inputs, outputs and the workspace.  All calls return a pl_status.
 *
 * Each entry point names the reference interface it replaces (paths inside
 * MiguelMonteiro/permutohedral_lattice).
 */
#ifndef PL_LATTICE_H
#define PL_LATTICE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum pl_status {
    PL_OK = 0,
    PL_INVALID_ARGUMENT = 1,    /* null pointer, negative size, size beyond 32-bit indexing */
    PL_UNSUPPORTED_DIMS = 2,    /* (pd, vd) without a compiled instantiation; see pl_supported */
    PL_WORKSPACE_TOO_SMALL = 3, /* workspace_bytes below pl_workspace_bytes for these sizes */
    PL_CAPACITY_EXCEEDED = 4,   /* more lattice entries than max_entries allowed (device-side) */
    PL_CUDA_ERROR = 5,          /* a CUDA runtime call failed; see pl_last_cuda_error */
    PL_INTERNAL_ERROR = 6       /* a bounded device loop gave up (should not happen) */
} pl_status;

/* Accumulation order of the splat stage. */
typedef enum pl_mode {
    PL_MODE_ATOMIC = 0,        /* floating-point reductions; sums differ run to run in the last bits */
    PL_MODE_DETERMINISTIC = 1  /* sorted, segmented reduction with exact (64-bit fixed-point) sums:
                                  bitwise reproducible; finite inputs, grid 2^-36 of max(|input|, 1) */
} pl_mode;

/* Counters read back from a workspace after a call (pl_lattice_stats). */
typedef struct pl_stats {
    int64_t num_vertices;  /* distinct lattice vertices over the whole batch */
    int64_t num_entries;   /* tile-local vertex entries (>= num_vertices) */
    int64_t table_slots;   /* hash table capacity chosen on the device for this call (direct indexing: the
                              dense index's slot count rounded up to a power of two) */
    int32_t device_status; /* pl_status recorded by the kernels (PL_OK, PL_CAPACITY_EXCEEDED, ...) */
    int32_t direct_index;  /* 1: vertices were located by direct indexing (spatial-only call), 0: hash table */
    int64_t max_entries;   /* the entry bound the workspace was laid out for (the worst case if the call passed 0):
                              what pl_export_lattice and pl_lattice_apply_f32 must be given again */
} pl_stats;

/* 1 if position dimension pd and value dimension vd (= input channels + 1) can be filtered.
 * Replaces the build-time SPATIAL_DIMS / INPUT_CHANNELS / REFERENCE_CHANNELS selection of
 * src/LatticeFilterKernel.cu:30-38,87-100 (one compiled pair, LOG(FATAL) otherwise). */
int pl_supported(int pd, int vd);

const char* pl_strerror(int status);

/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
const char* pl_last_cuda_error(void);

/* Bytes of device workspace for `batch` items of `n` points each.  spatial_dims (HOST array, product
 * n) must be the one later given to pl_lattice_filter_f32; pass NULL for pl_filter_f32 (points are
 * then tiled in index order).  max_entries bounds the lattice entries the call may create over the
 * whole batch; 0 means the worst case batch*n*(pd+1), which can never overflow.  A smaller bound (a
 * previous call's pl_stats.num_entries for similar data, with some margin) shrinks everything that
 * is indexed by entry or by vertex, which is most of the workspace; a call that outgrows it reports
 * PL_CAPACITY_EXCEEDED through pl_lattice_stats, fills its output with NaN and can be repeated with a
 * larger bound.  mode: the pl_mode the workspace will serve; PL_MODE_DETERMINISTIC adds the 64-bit
 * sums (a workspace sized for it serves both modes).  Replaces the scratch allocations of
 * PermutohedralLatticeGPU's constructor (src/PermutohedralLatticeGPU.cuh:434-451) and
 * src/DeviceMemoryAllocator.h:47-120. */
int pl_workspace_bytes(int batch, int n, int pd, int vd, int n_spatial_dims, const int* spatial_dims,
                       int64_t max_entries, int mode, size_t* bytes);

/* positions[n*pd] (device) <- feature vectors: for each spatial dimension s (row-major pixel order,
 * last dimension fastest) coordinate / spatial_std, then reference[c] / feature_std.
 * spatial_dims is a HOST array.  reference may be NULL when n_reference_channels == 0.
 * Replaces ComputeKernel<GPUDevice,T>::operator() (src/LatticeFilterKernel.h:40-54,
 * src/LatticeFilterKernel.cu:44-68) and compute_bilateral_kernel_gpu / compute_spatial_kernel_gpu
 * (Tests/bilateral_filter_gpu.h:8-19, Tests/PermutohedralLatticeGPU.cu:19-42). */
int pl_compute_positions_f32(const float* reference, float* positions, int n,
                             int n_reference_channels, int n_spatial_dims, const int* spatial_dims,
                             float spatial_std, float feature_std, void* stream);

/* output[batch*n*(vd-1)] <- lattice filter of input[batch*n*(vd-1)] at positions[batch*n*pd]
 * (all device, item-major, channels last).  Each batch item is an independent lattice.
 * reverse != 0 runs the blur axes pd..0 (the reference's gradient definition).
 * Replaces LatticeFilter<GPUDevice,T>::operator() (src/LatticeFilterKernel.h:28-38,
 * src/LatticeFilterKernel.cu:75-101), PermutohedralLatticeGPU::filter
 * (src/PermutohedralLatticeGPU.cuh:454-479) and lattice_filter_gpu (Tests/PermutohedralLatticeGPU.cu:6-16),
 * one call per batch instead of one per item. */
int pl_filter_f32(float* output, const float* input, const float* positions, int batch, int n,
                  int pd, int vd, int reverse, void* workspace, size_t workspace_bytes,
                  int64_t max_entries, int mode, void* stream);

/* The whole op on device tensors input[batch, *spatial_dims, n_input_channels] and
 * reference[batch, *spatial_dims, n_reference_channels]: features are built on the fly (never
 * written to memory).  bilateral != 0: pd = n_spatial_dims + n_reference_channels, coordinates
 * divided by theta_alpha, reference channels by theta_beta.  bilateral == 0: pd = n_spatial_dims,
 * coordinates divided by theta_gamma, reference unused (may be NULL).  spatial_dims is a HOST array.
 * Replaces LatticeFilterOp<GPUDevice,T>::Compute (src/LatticeFilterKernel.cpp:98-181) for the
 * op registered at src/LatticeFilterKernel.cpp:30-43. */
int pl_lattice_filter_f32(float* output, const float* input, const float* reference, int batch,
                          int n_spatial_dims, const int* spatial_dims, int n_input_channels,
                          int n_reference_channels, int bilateral, float theta_alpha,
                          float theta_beta, float theta_gamma, int reverse, void* workspace,
                          size_t workspace_bytes, int64_t max_entries, int mode, void* stream);

/* The same filter in two halves, for callers that filter several value tensors through ONE reference
 * (forward and backward of a layer, the iterations of CRF mean-field inference: the use the reference
 * library was written for, README.md:15-16, which rebuilds its lattice on every call,
 * src/LatticeFilterKernel.cpp:79, src/LatticeFilterKernel.cu:88).
 * pl_lattice_build*_f32 constructs the lattice of a batch in `workspace` (entries, vertices, neighbour
 * table, per-point records); pl_lattice_apply_f32 then splats, blurs and slices `input` through it and
 * may be called any number of times, with any number of channels up to max_value_dim - 1, forward or
 * reverse, while the workspace is left untouched in between.  build + apply gives bit-for-bit what
 * pl_lattice_filter_f32 / pl_filter_f32 give (in deterministic mode; in atomic mode up to the order of
 * the sums).  The geometry arguments of apply (batch, n, pd, spatial_dims or NULL for a lattice built
 * from positions, max_entries) must repeat those of the build; workspace_bytes must cover
 * pl_workspace_bytes(..., vd = max_value_dim, ...).  A lattice built this way also keeps every tile's
 * splats sorted by vertex, so that no apply sorts them again (the build takes a quarter longer for it,
 * every splat a fifth less); apply on a workspace that no pl_lattice_build*_f32 prepared (the one a
 * pl_lattice_filter_f32 call left, say) reports PL_INVALID_ARGUMENT through pl_lattice_stats and fills
 * the output with NaN. */
int pl_lattice_build_f32(const float* reference, int batch, int n_spatial_dims, const int* spatial_dims,
                         int n_reference_channels, int bilateral, float theta_alpha, float theta_beta,
                         float theta_gamma, int max_value_dim, void* workspace, size_t workspace_bytes,
                         int64_t max_entries, void* stream);
int pl_lattice_build_positions_f32(const float* positions, int batch, int n, int pd, int max_value_dim,
                                   void* workspace, size_t workspace_bytes, int64_t max_entries, void* stream);
int pl_lattice_apply_f32(float* output, const float* input, int n_input_channels, int reverse, int mode, int batch,
                         int n, int pd, int n_spatial_dims, const int* spatial_dims, void* workspace,
                         size_t workspace_bytes, int64_t max_entries, void* stream);

/* The op for callers that must not allocate device memory and have no buffer to lend: a plugin
 * loaded into a host application whose memory pool already owns the GPU's memory, or a service that
 * forbids allocation calls once it is running.  Same arguments and results as
 * pl_lattice_filter_f32 (atomic mode), but the scratch is an array built into the library image:
 * PL_STATIC_SCRATCH_BYTES on every GPU that loads the library, held until the process exits.
 * This entry point has no counterpart in the reference.
 *  - It calls no cudaMalloc / cudaFree and no allocating library routine.
 *  - A call whose pl_workspace_bytes exceeds PL_STATIC_SCRATCH_BYTES returns
 *    PL_WORKSPACE_TOO_SMALL before launching anything (pl_last_cuda_error then holds the two sizes);
 *    a smaller max_entries shrinks the need.  Whether the lattice stayed within that max_entries is
 *    known only on the device: read it with pl_lattice_stats(NULL, &stats, stream) and check
 *    stats.device_status (on PL_CAPACITY_EXCEEDED the output holds NaN).
 *  - The first call on each device looks up the scratch's device address (the device must be
 *    current, as for every call); make that first call outside any stream capture.
 *  - All calls on a device share the one scratch, which keeps the previous call's contents; each call
 *    clears what it needs zeroed.  Two calls that overlap on the GPU (different streams, different
 *    host threads) race on it: serialise them. */
#define PL_STATIC_SCRATCH_BYTES (64u << 20)
int pl_lattice_filter_f32_noalloc(float* output, const float* input, const float* reference, int batch,
                                  int n_spatial_dims, const int* spatial_dims, int n_input_channels,
                                  int n_reference_channels, int bilateral, float theta_alpha,
                                  float theta_beta, float theta_gamma, int reverse, int64_t max_entries,
                                  void* stream);

/* T = double.  The reference registers its op and instantiates its functors for double as well as
 * float (src/LatticeFilterKernel.cpp:196-197,207-208, src/LatticeFilterKernel.cu:107-108); these
 * entry points are the double counterparts of pl_workspace_bytes, pl_compute_positions_f32,
 * pl_filter_f32, pl_lattice_filter_f32 and pl_export_lattice, with the same argument meaning.  The
 * geometry follows the reference's arithmetic for T = double operation by operation (including the
 * one product of the elevation step that it keeps in a float, src/PermutohedralLatticeCPU.h:226), so
 * vertex keys and barycentric weights equal the reference CPU path bit for bit; the splat sums are
 * double-precision reductions whose order varies from run to run.  A workspace sized by
 * pl_workspace_bytes_f64 serves the double calls only.  The build / apply split, the deterministic
 * mode and the no-allocation entry exist for float only. */
int pl_workspace_bytes_f64(int batch, int n, int pd, int vd, int n_spatial_dims, const int* spatial_dims,
                           int64_t max_entries, size_t* bytes);
int pl_compute_positions_f64(const double* reference, double* positions, int n, int n_reference_channels,
                             int n_spatial_dims, const int* spatial_dims, double spatial_std,
                             double feature_std, void* stream);
int pl_filter_f64(double* output, const double* input, const double* positions, int batch, int n, int pd,
                  int vd, int reverse, void* workspace, size_t workspace_bytes, int64_t max_entries,
                  void* stream);
int pl_lattice_filter_f64(double* output, const double* input, const double* reference, int batch,
                          int n_spatial_dims, const int* spatial_dims, int n_input_channels,
                          int n_reference_channels, int bilateral, double theta_alpha, double theta_beta,
                          double theta_gamma, int reverse, void* workspace, size_t workspace_bytes,
                          int64_t max_entries, void* stream);
int pl_export_lattice_f64(const void* workspace, const double* positions, const double* reference, int batch,
                          int n, int pd, int vd, int n_spatial_dims, const int* spatial_dims,
                          int n_reference_channels, double spatial_std, double feature_std, int64_t max_entries,
                          int64_t max_vertices, int16_t* vertex_keys, int32_t* vertex_item,
                          int32_t* pixel_vertex, double* pixel_weight, void* stream);

/* Profiling aid: the next pl_filter_f32 / pl_lattice_filter_f32 call made by this host thread records
 * the PL_NUM_STAGE_EVENTS cudaEvent_t handles of stage_events[] on its stream at the stage
 * boundaries (start, after build, after index, after splat, after blur, after slice), then forgets
 * them.  The array must stay valid until that call returns.  NULL cancels.
 * The reference only times whole calls with std::clock (Tests/test_bilateral_gpu.cpp:32-36). */
#define PL_NUM_STAGE_EVENTS 6
int pl_profile_next_call(void** stage_events);

/* The pointwise half of one dense-CRF mean-field update, in one pass over memory (all pointers device,
 * [n_points][n_labels] floats, channels last as everywhere else):
 *   q_out = softmax over labels ( -unaries - (bilateral_weight * q_bilateral + spatial_weight * q_spatial) @ compatibility )
 * q_bilateral / q_spatial are the current label distributions filtered through the appearance and the
 * smoothness kernel (pl_lattice_apply_f32 on two lattices built once per image); compatibility is
 * [n_labels][n_labels] row-major, or NULL for the Potts model (1 - identity).  n_labels <= 128.
 * q_out must not overlap the inputs.  No counterpart in the reference: it ships no CRF code, its README
 * (README.md:15-16) names CRF-as-RNN as the user the filter was written for; this is the step either
 * side of the filter in that user. */
int pl_crf_update_f32(float* q_out, const float* unaries, const float* q_bilateral, const float* q_spatial,
                      const float* compatibility, float bilateral_weight, float spatial_weight,
                      int64_t n_points, int n_labels, void* stream);

/* Number of kernels the library has launched in this process so far (filter stages and pl_crf_update_f32;
 * memsets, copies and event records are not counted).  The difference across a region is the number
 * of kernels that region launched.  No counterpart in the reference. */
unsigned long long pl_launch_count(void);

/* Spatial-only calls (bilateral == 0: the features are the grid coordinates divided by theta_gamma,
 * src/LatticeFilterKernel.cpp:137-142, compute_spatial_kernel_gpu in Tests/PermutohedralLatticeGPU.cu:33-42)
 * locate their vertices by direct indexing instead of hashing whenever the dense index fits the
 * workspace's table region: the region of the lattice such a call can touch is known from the grid's
 * size alone.  Results are identical either way.  This process-wide developer switch turns that path
 * off (enable == 0) or back on, for A/B timing and tests; it returns the previous setting.  The
 * reference hashes always (src/PermutohedralLatticeGPU.cuh:76-143). */
int pl_debug_direct_index(int enable);

/* min_entries <- the smallest max_entries whose workspace lets a spatial-only call on this grid locate its
 * vertices by direct indexing (the dense index lives in the table region, whose size follows max_entries), or
 * 0 when the grid cannot be indexed directly at all.  For callers that pass a max_entries of their own: a
 * smaller bound still works, the call then hashes.  The reference hashes always
 * (src/PermutohedralLatticeGPU.cuh:76-143). */
int pl_direct_index_min_entries(int batch, int n_spatial_dims, const int* spatial_dims, float theta_gamma,
                                int64_t* min_entries);

/* Copies the counters of the last call that used `workspace` to the host.  SYNCHRONISES `stream`.
 * workspace == NULL reads the counters of the last pl_lattice_filter_f32_noalloc call on the current
 * device (its scratch is inside the library, so that caller has no pointer to pass).
 * Returns PL_OK when read; the call's own outcome is stats->device_status.  A call whose device_status
 * is not PL_OK (for instance PL_CAPACITY_EXCEEDED under a max_entries that was too small) has filled
 * its whole output with NaN: a failed call never leaves bytes that could pass for a result.
 * No counterpart in the reference (it prints or exits: src/PermutohedralLatticeGPU.cuh:49-55,442-445). */
int pl_lattice_stats(const void* workspace, pl_stats* stats, void* stream);

/* Lattice structure of the last call that used `workspace`, for verification (all outputs device,
 * any may be NULL): vertex_keys[num_vertices*pd] int16 and vertex_item[num_vertices] (batch item of
 * each vertex), pixel_vertex[batch*n*(pd+1)] (vertex index of each point's simplex corners,
 * remainder ascending) and pixel_weight[batch*n*(pd+1)] (barycentric weights).  The positions /
 * reference arguments must be the ones given to that call (pass positions for pl_filter_f32,
 * reference + geometry for pl_lattice_filter_f32; the unused one NULL).  vertex arrays must hold
 * max_vertices rows; rows beyond num_vertices are left untouched.
 * Corresponds to HashTableCPU::getKeys and the MatrixEntry records
 * (src/PermutohedralLatticeCPU.h:153-154,187-191). */
int pl_export_lattice(const void* workspace, const float* positions, const float* reference,
                      int batch, int n, int pd, int vd, int n_spatial_dims, const int* spatial_dims,
                      int n_reference_channels, float spatial_std, float feature_std,
                      int64_t max_entries, int64_t max_vertices, int16_t* vertex_keys,
                      int32_t* vertex_item, int32_t* pixel_vertex, float* pixel_weight,
                      void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PL_LATTICE_H */
