/* picasso_b200.h — C ABI of libpicasso_b200.so: the mesh-convolution operators of
 * PicassoPlus (vertex->facet, facet->facet, facet->vertex; forward and backward), the
 * spherical-harmonic basis, and the adjacency they need, as CUDA kernels for sm_100a.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer owned by the caller; no call allocates or frees
 *     device memory.  Scratch memory is passed in as `workspace` and sized by the matching
 *     `*_workspace_bytes` query.  Two fixed resources belong to the library itself: a 4 MiB
 *     `__device__` array in the library image (scratch of pb200_vertex2facet_backward_static,
 *     resident on every GPU that loads the library) and one small block of pinned, mapped HOST
 *     memory for the asynchronous error words below, allocated by the first facet2facet call of
 *     the process that takes a tensor-core path -- make that first call outside stream capture.
 *   - features are fp32, row-major, contiguous; indices are int32.
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).  All work
 *     is enqueued on it; no call synchronises unless its comment says so.
 *   - return value: PB200_OK (0) or a negative PB200_E* code; pb200_last_error() returns
 *     a human-readable message for the calling thread's last failure.  Nothing throws,
 *     prints or exits.
 *   - output buffers are fully written by the call (no need to zero them first), with the
 *     values the reference writes into its zero-initialised outputs.
 *   - results are run-to-run deterministic: no floating-point atomics are used.
 *
 * Citations name files of the reference tree (EnyaHermite/PicassoPlus).
 */
#ifndef PICASSO_B200_H
#define PICASSO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PB200_OK            0
#define PB200_EINVAL       -1   /* bad size / null pointer / unsupported shape            */
#define PB200_EWORKSPACE   -2   /* workspace missing or too small                          */
#define PB200_ECUDA        -3   /* a CUDA runtime call or launch failed                    */
#define PB200_EINDEX       -4   /* an index array holds an out-of-range value              */

/* contraction precision for facet2facet (fp32 accumulation in every mode) */
#define PB200_PREC_FP32     0   /* every operand as bf16 hi + bf16 lo, three tensor-core products
                                   per term (FFMA where the shape has no tensor-core kernel):
                                   about 1e-5 relative error, meets the 1e-4 gate            */
#define PB200_PREC_TF32     1   /* tf32 operands on the tensor cores                       */
#define PB200_PREC_BF16     2   /* bf16 operands on the tensor cores (2e-2 relative gate)  */
#define PB200_PREC_FP32_FFMA 3  /* fp32 FFMA path (no tensor cores), every shape            */
#define PB200_PREC_FP32_TF32X3 4 /* every operand as tf32 hi + tf32 lo, three products per term:
                                   about 2e-6 relative error, as close to fp64 as the reference's
                                   own FFMA kernels; about a quarter slower than PB200_PREC_FP32 */

int         pb200_version(void);
const char* pb200_last_error(void);
/* number of kernel launches issued by this library in this process so far */
int64_t     pb200_launch_count(void);

/* ---- asynchronous errors of the tensor-core kernels ------------------------------------
 * Every wait inside the facet2facet tensor-core kernels is bounded (about one second of GPU
 * clocks; such a wait can only run out if the GPU is preempted for that long or a kernel has a
 * defect).  A kernel whose wait runs out unwinds, frees its tensor memory and raises a word in
 * mapped host memory, one word per device.  The call that launched it has already returned
 * PB200_OK and its outputs are invalid.  While the word of the current device is raised, every
 * later facet2facet call on that device fails with PB200_ECUDA.  pb200_async_error() reads the
 * word of the current device (0 = none; 1/2/3 = facet2facet forward / input-gradient /
 * filter-gradient kernel, 4 = fused operator + pointwise kernel) -- call it after synchronising the stream to learn whether the step's results are
 * good; pb200_clear_async_error() re-arms the device.  pb200_set_wait_budget() changes the
 * budget of later launches (clocks; <= 0 restores the default).  A cudaDeviceReset() by the host
 * invalidates nothing here, but it does invalidate the device address that
 * pb200_vertex2facet_backward_static caches: do not reset a device between calls of that entry. */
int  pb200_async_error(void);
void pb200_clear_async_error(void);
void pb200_set_wait_budget(int64_t clocks);
/* Test switch: while on, the forward kernel's filter stream issues no copies, so the kernel's
 * waits run out after the wait budget and the error path above is exercised.  Never set it
 * outside a test. */
void pb200_test_silence_filter_stream(int on);

/* ---- per-kernel timing (for benchmarks) -------------------------------------------
 * When enabled, every launch is bracketed by CUDA events on its stream.  pb200_prof_read
 * synchronises those events and fills up to `cap` records sorted by total time; it
 * returns the number of distinct kernels seen.  Off by default. */
typedef struct { char name[48]; int64_t launches; double total_ms; } pb200_prof_record;
void pb200_prof_enable(int on);
void pb200_prof_reset(void);
int  pb200_prof_read(pb200_prof_record* out, int cap);

/* ---- adjacency ----------------------------------------------------------------------
 * nfCount[vtMap[face[f][j]]] += 1 for every face corner whose mapped id is >= 0.
 * Replaces count_vertex_adjface (picasso/mesh/pi_modules/source/decimate_gpu.cu:813-836,
 * binding decimate.cpp:132-160).  vtMap may be NULL (identity).  nfCount: NvOut ints. */
int pb200_count_vertex_adjface(int64_t Nf, int64_t NvIn, int64_t NvOut, const int32_t* face,
                               const int32_t* vtMap, int32_t* nfCount, void* stream);

/* Vertex -> incident face-corner lists in CSR form, keyed by the OUTPUT vertex
 * vo = vtMap[face[f][j]] (corners with vo < 0 are dropped).  rowptr has NvOut+1 entries;
 * entries[rowptr[v] .. rowptr[v+1]) hold (f << 2 | j) in ascending order, so every
 * segmented reduction over a row has one fixed order.  rowptr[v+1]-rowptr[v] equals the
 * reference's nfCount[v] bit for bit.  `entries` needs 3*Nf ints.  `status` (one int,
 * device) is set to 0, or to PB200_EINDEX if a face id is outside [0,NvIn) or a vtMap
 * value is outside [-1,NvOut) (such corners are skipped, never dereferenced).
 * The reference has no such structure: it scatters with float atomics instead
 * (picasso/mesh/pi_modules/source/mesh_conv3d_gpu.cu:215,326). */
size_t pb200_vertex_csr_workspace_bytes(int64_t Nf, int64_t NvOut);
int pb200_build_vertex_csr(int64_t Nf, int64_t NvIn, int64_t NvOut, const int32_t* face,
                           const int32_t* vtMap, int32_t* rowptr, int32_t* entries,
                           int32_t* status, void* workspace, size_t workspace_bytes, void* stream);

/* ---- vertex2facet -------------------------------------------------------------------
 * output[f, c*r+m] = sum_{k<3} filter[k,c,m] * input[face[f,k], c]
 * Replaces vertex2facetConv3dLauncher (mesh_conv3d_gpu.cu:176-195,261-266; binding
 * mesh_conv3d.cpp:123-152).  input (Nv,C), filter (3,C,r), face (Nf,3), output (Nf,C*r). */
int pb200_vertex2facet_forward(int64_t Nf, int64_t Nv, int C, int r, const float* input,
                               const float* filter, const int32_t* face, float* output, void* stream);

/* gradInput[v,c]  = sum_{(f,k): face[f,k]=v} sum_m gradOutput[f,c*r+m] * filter[k,c,m]
 * gradFilter[k,c,m] = sum_f gradOutput[f,c*r+m] * input[face[f,k], c]
 * Replaces vertex2facetConv3dGradLauncher (mesh_conv3d_gpu.cu:201-260,267-290; binding
 * mesh_conv3d.cpp:153-188).  rowptr/entries: CSR built with vtMap = NULL over Nv vertices. */
size_t pb200_vertex2facet_backward_workspace_bytes(int64_t Nf, int64_t Nv, int C, int r);
int pb200_vertex2facet_backward(int64_t Nf, int64_t Nv, int C, int r, const float* gradOutput,
                                const float* input, const float* filter, const int32_t* face,
                                const int32_t* rowptr, const int32_t* entries,
                                float* gradInput, float* gradFilter,
                                void* workspace, size_t workspace_bytes, void* stream);

/* Allocation-free variant of pb200_vertex2facet_backward.  It has no counterpart in the
 * reference.  It is for callers that cannot obtain device memory at call time: code that
 * runs where the embedding framework's allocator is frozen or off limits, callbacks with a
 * fixed memory budget, hosts that may not call cudaMalloc after start-up.  The scratch the
 * backward pass needs (per-block filter-gradient partials) is a fixed array inside the
 * library image, pb200_vertex2facet_backward_static_max_bytes() = 4 MiB, resident on every
 * GPU that loads the library until the process exits.  The caller still passes all inputs
 * and outputs.
 *   - limit: shapes whose pb200_vertex2facet_backward_workspace_bytes() exceed the array
 *     are refused with PB200_EWORKSPACE and a message that names both sizes (e.g.
 *     C*r = 128 needs 1.8 MB on a 148-SM part; C*r above ~290 does not fit).
 *   - the first call on each device looks up the array's device address (one
 *     cudaGetSymbolAddress, with that device current); make that first call outside any
 *     stream capture.  No call allocates or frees memory.
 *   - all calls on one device share the array: two calls that overlap on the GPU (different
 *     streams, or different threads without ordering) race on it.  Calls that are ordered
 *     on one stream are safe.  Nothing in the array needs clearing between calls: each call
 *     writes every partial before it reads it; the array keeps the last call's partials.
 *   - results are bit-identical to pb200_vertex2facet_backward for the same shape. */
size_t pb200_vertex2facet_backward_static_max_bytes(void);
int pb200_vertex2facet_backward_static(int64_t Nf, int64_t Nv, int C, int r, const float* gradOutput,
                                       const float* input, const float* filter, const int32_t* face,
                                       const int32_t* rowptr, const int32_t* entries,
                                       float* gradInput, float* gradFilter, void* stream);

/* ---- facet2vertex -------------------------------------------------------------------
 * w[f,co] = sum_k coeff[f,k]*filter[k,c,m];
 * output[vo,co] = (sum over corners (f,j) with vtMap[face[f,j]] = vo of w[f,co]*input[f,c])
 *                 / nfCount[vo];  rows no corner maps to are 0.
 * Replaces facet2vertexConv3dLauncher (mesh_conv3d_gpu.cu:299-329,428-433; binding
 * mesh_conv3d.cpp:33-74).  input (Nf,C), filter (K,C,r), coeff (Nf,K), nfCount (NvOut),
 * output (NvOut,C*r); rowptr/entries: CSR built with the same face/vtMap.  The kernels
 * never read vtMap or face here (the CSR carries them).  Workspace: one (Nf, C) fp32 array
 * for the per-face products w*input (0 bytes for shapes that take the scalar path). */
size_t pb200_facet2vertex_forward_workspace_bytes(int64_t Nf, int C, int r, int K);
int pb200_facet2vertex_forward(int64_t Nf, int64_t NvOut, int C, int r, int K, const float* input,
                               const float* filter, const float* coeff, const int32_t* nfCount,
                               const int32_t* rowptr, const int32_t* entries, float* output,
                               void* workspace, size_t workspace_bytes, void* stream);

/* gt[f,co] = sum_{j<3, vo_j>=0} gradOutput[vo_j,co] / nfCount[vo_j];
 * gradInput[f,c] = sum_m gt[f,co]*w[f,co];  gradFilter[k,c,m] = sum_f coeff[f,k]*input[f,c]*gt[f,co]
 * Replaces facet2vertexConv3dGradLauncher (mesh_conv3d_gpu.cu:338-426,434-458; binding
 * mesh_conv3d.cpp:75-122).  vtMap may be NULL (identity). */
size_t pb200_facet2vertex_backward_workspace_bytes(int64_t Nf, int C, int r, int K);
int pb200_facet2vertex_backward(int64_t Nf, int64_t NvIn, int64_t NvOut, int C, int r, int K,
                                const float* gradOutput, const float* input, const float* filter,
                                const float* coeff, const int32_t* face, const int32_t* nfCount,
                                const int32_t* vtMap, float* gradInput, float* gradFilter,
                                void* workspace, size_t workspace_bytes, void* stream);

/* ---- operator + pointwise stage in one kernel (module-level fusion) ----------------------
 * output[row, co] = act( sum_c feat[row, c] * depthWeights[c, co] + bias[co] ), act = ReLU if relu != 0,
 * where feat is the operator's output for depth multiplier 1 and is never written to memory:
 *   vertex2facet:  feat = pb200_vertex2facet_forward(input, filter (3,C,1), face)           rows = faces
 *   facet2vertex:  feat = pb200_facet2vertex_forward(input, filter (K,C,1), coeff, CSR)     rows = output vertices
 * The product runs on the tensor cores (tcgen05, fp32 accumulation): PB200_PREC_FP32 = bf16 hi+lo
 * operands, three products per term (about 1e-5 relative); PB200_PREC_BF16 = bf16 operands.
 * Replaces, inside V2FConv3d.forward / F2VConv3d.forward (picasso/mesh/layers.py:109-120,166-175), the
 * sequence operator -> torch.matmul(., depth_weights) -> + biases -> ReLU and the (rows, C) round trip
 * through memory between them.  depthWeights (C, Cout) row-major, bias (Cout) or NULL, C % 8 == 0,
 * input / filter / workspace 16-byte aligned.  The facet2vertex workspace also holds the per-face
 * products (Nf, C).  The first call of the process allocates the asynchronous error words (see above). */
size_t pb200_vertex2facet_pointwise_workspace_bytes(int C, int precision);
int pb200_vertex2facet_pointwise_forward(int64_t Nf, int64_t Nv, int C, int Cout, const float* input,
                                         const float* filter, const int32_t* face, const float* depthWeights,
                                         const float* bias, int relu, float* output, int precision,
                                         void* workspace, size_t workspace_bytes, void* stream);
size_t pb200_facet2vertex_pointwise_workspace_bytes(int64_t Nf, int C, int precision);
int pb200_facet2vertex_pointwise_forward(int64_t Nf, int64_t NvOut, int C, int K, int Cout, const float* input,
                                         const float* filter, const float* coeff, const int32_t* nfCount,
                                         const int32_t* rowptr, const int32_t* entries,
                                         const float* depthWeights, const float* bias, int relu, float* output,
                                         int precision, void* workspace, size_t workspace_bytes, void* stream);

/* output[row, co] = act(sum_c rows[row, c] * weights[c, co] + bias[co]) on the tensor cores: the pointwise layer of
 * the reference's networks (PerItemConv3d, picasso/mesh/layers.py:198-240: torch.matmul, + biases, activation as
 * separate kernels).  rows (Nrows, C), C a multiple of 8; weights (C, Cout); bias (Cout) or NULL; relu 0/1.
 * Workspace as pb200_masked_rows_matmul_workspace_bytes(C, precision).  Its backward is the next two entries. */
int pb200_rows_pointwise_forward(int64_t Nrows, int C, int Cout, const float* rows, const float* weights, const float* bias,
                                 int relu, float* output, int precision, void* workspace, size_t workspace_bytes,
                                 void* stream);
/* Backward of the pointwise stage on the tensor cores (no counterpart in the reference, whose modules leave it
 * to autograd): output[row, co] = sum_c g[row, c] * weights[c, co] with g = rows where mask > 0, else 0
 * (mask = the stage's activated output; NULL = no activation).  rows, mask (Nrows, C), C a multiple of 8;
 * weights (C, Cout) row-major -- pass depth_weights transposed to get the gradient of the operator output;
 * maskedRows (Nrows, C), may be NULL, receives g itself (needed for the weight and bias gradients).
 * Precision PB200_PREC_FP32 (bf16 hi + lo operands, about 1e-5 relative) or PB200_PREC_BF16. */
size_t pb200_masked_rows_matmul_workspace_bytes(int C, int precision);
int pb200_masked_rows_matmul(int64_t Nrows, int C, int Cout, const float* rows, const float* mask, const float* weights,
                             float* output, float* maskedRows, int precision, void* workspace, size_t workspace_bytes,
                             void* stream);

/* out[m, n] = sum over rows of A[row, m] * B[row, n] and, if colsum is not NULL, colsum[n] = sum over rows of
 * B[row, n]: the weight and bias gradients of a pointwise stage (A = its input rows, B = the masked upstream
 * gradient), which the reference's modules leave to autograd (an fp32 GEMM whose contraction runs over millions
 * of rows).  A (Nrows, M), B (Nrows, N) row-major, M and N multiples of 4, 16-byte aligned; out (M, N).
 * Tensor cores with bf16 hi + lo operands (PB200_PREC_FP32, about 1e-5 relative) or bf16 (PB200_PREC_BF16);
 * at most 4096 rows go through one accumulator chain, the partial results are added in a fixed order. */
size_t pb200_rows_contract_workspace_bytes(int64_t Nrows, int M, int N);
int pb200_rows_contract(int64_t Nrows, int M, int N, const float* A, const float* B, float* out, float* colsum,
                        int precision, void* workspace, size_t workspace_bytes, void* stream);

/* ---- facet2facet --------------------------------------------------------------------
 * A[f,d,ci] = (1/T_f) sum_{k in samples(f)} bary[k,d]*input[k,ci];
 * output[f,co] = sum_{d,ci} A[f,d,ci]*filter[co,ci,d];  samples(f) = rows
 * numInterior[f-1] .. numInterior[f]-1 (numInterior = inclusive cumulative sample count).
 * Replaces facet2facetConv3dLauncher (mesh_conv3d_gpu.cu:6-37,136-143; binding
 * mesh_conv3d.cpp:192-228).  input (NiK,Cin), filter (Cout,Cin,F), bary (NiK,F),
 * output (Nf,Cout).  F <= 50 as in the reference (mesh_conv3d.cpp:211).
 * numInterior is trusted, as in the reference: it must be non-decreasing, lie in [0, NiK] and end
 * at NiK; pb200_check_num_interior verifies that on the device (status = 0 or PB200_EINDEX; run it
 * once per numInterior array, e.g. alongside the CSR build, and read `status` after a sync). */
int pb200_check_num_interior(int64_t Nf, int64_t NiK, const int32_t* numInterior, int32_t* status, void* stream);
size_t pb200_facet2facet_forward_workspace_bytes(int64_t Nf, int64_t NiK, int Cin, int Cout, int F, int precision);
int pb200_facet2facet_forward(int64_t Nf, int64_t NiK, int Cin, int Cout, int F, const float* input,
                              const float* filter, const float* bary, const int32_t* numInterior,
                              float* output, int precision,
                              void* workspace, size_t workspace_bytes, void* stream);

/* facet2facet forward for faces that have exactly one sample each (numInterior = 1, 2, ..., Nf is implied):
 *   output[f,co] = sum_d weights[f,d] * sum_ci input[f,ci]*filter[co,ci,d],
 * input (Nf,Cin), weights (Nf,F), filter (Cout,Cin,F), output (Nf,Cout).  Same result as pb200_facet2facet_forward
 * with that numInterior; on the tensor cores it runs as a plain product over the input rows with the weighted sum
 * over d in the epilogue (the input-gradient kernel with the channel roles exchanged), which needs no face operand
 * of F*Cin products.  With pb200_face_mean_rows this is the forward pass of "one row per face shared by its
 * samples"; the matching backward is pb200_facet2facet_backward over (input, weights, numInterior = 1..Nf).
 * weightsPadded (may be NULL): the pb200_pad_rows copy of weights; given, the call does not pad weights itself.
 * No counterpart inside the reference's extension. */
size_t pb200_facet2facet_one_sample_forward_workspace_bytes(int64_t Nf, int Cin, int Cout, int F, int precision);
int pb200_facet2facet_one_sample_forward(int64_t Nf, int Cin, int Cout, int F, const float* input, const float* filter,
                                         const float* weights, const float* weightsPadded, float* output, int precision,
                                         void* workspace, size_t workspace_bytes, void* stream);

/* gradInput[k,ci] = (1/T_f) sum_d bary[k,d] * sum_co gradOutput[f,co]*filter[co,ci,d];
 * gradFilter[co,ci,d] = sum_f gradOutput[f,co]*A[f,d,ci]
 * Replaces facet2facetConv3dGradLauncher (mesh_conv3d_gpu.cu:45-135,144-168; binding
 * mesh_conv3d.cpp:229-269).  The tensor-core modes need gradOutput, input, bary and the
 * workspace on 16-byte boundaries (PB200_EINVAL otherwise); the workspace holds the filter
 * image of the input-gradient kernel, the per-chunk filter-gradient partials and, when F is
 * not a multiple of 4, a copy of bary with rows padded to 4 floats. */
size_t pb200_facet2facet_backward_workspace_bytes(int64_t Nf, int64_t NiK, int Cin, int Cout, int F, int precision);
int pb200_facet2facet_backward(int64_t Nf, int64_t NiK, int Cin, int Cout, int F, const float* gradOutput,
                               const float* input, const float* filter, const float* bary,
                               const int32_t* numInterior, float* gradInput, float* gradFilter,
                               int precision, void* workspace, size_t workspace_bytes, void* stream);

/* The tensor-core kernels read the rows of bary 16 bytes at a time; when F is not a multiple of 4 they work on a copy
 * with rows padded to pb200_padded_row_floats(F) floats (pad columns zero) that every call makes in its workspace.  A
 * caller that uses the same bary for several calls (forward and backward of a step, several steps) can make the copy once
 * with pb200_pad_rows (out: (N, pb200_padded_row_floats(F)), 16-byte aligned) and pass it as baryPadded; NULL = pad
 * inside the call as pb200_facet2facet_backward does.  Same results bit for bit. */
int pb200_padded_row_floats(int F);
int pb200_pad_rows(int64_t N, int F, const float* rows, float* out, void* stream);
int pb200_facet2facet_backward_padded(int64_t Nf, int64_t NiK, int Cin, int Cout, int F, const float* gradOutput,
                                      const float* input, const float* filter, const float* bary, const float* baryPadded,
                                      const int32_t* numInterior, float* gradInput, float* gradFilter,
                                      int precision, void* workspace, size_t workspace_bytes, void* stream);

/* ---- spherical-harmonic basis and triangle geometry -----------------------------------
 * out[i, 0..(L+1)^2) = real/imaginary spherical-harmonic components of xyz[i] projected
 * to the unit sphere, in the reference's column order, L <= 5.
 * Replaces SphHarmCoeff.__call__ (picasso/mesh/layers.py:341-356) with
 * torch_sph_harm_reorder (picasso/math_utils.py:10-62).  xyz (N,3) contiguous. */
int pb200_sph_harm_coeff(int64_t N, int L, const float* xyz, float* out, void* stream);

/* geometry[f] = [unit normal (3), plane intercept d, area].  Replaces
 * compute_triangle_geometry_ (picasso/mesh/pi_modules/decimate.py:70-85).  `vertex` has
 * `vstride` floats per row, of which the first three are xyz. */
int pb200_triangle_geometry(int64_t Nf, int64_t Nv, int vstride, const float* vertex,
                            const int32_t* face, float* geometry, void* stream);

/* Per-level preparation in one call: for every face the triangle geometry (as pb200_triangle_geometry;
 * `geometry` may be NULL), the normal the filter coefficients are taken from -- the geometric normal,
 * or with orient != 0 the normal flipped towards the origin as viewpoint
 * (picasso/networks/scene_seg.py:117-124: sign = sign(sum(-center*normal)), every sign above -1 set to
 * +1; `normals` (Nf,3) may be NULL) -- and coeff (Nf,(L+1)^2) = its spherical-harmonic basis (as
 * pb200_sph_harm_coeff); for the vertices nfCount (as pb200_count_vertex_adjface) and the vertex CSR
 * (as pb200_build_vertex_csr, same workspace size, same `status`).  The faces are read once: one
 * kernel does geometry, orientation, basis and corner counting.  Replaces, per mesh level, the
 * sequence compute_triangle_geometry_ (decimate.py:70-85), get_oriented_normals, SphHarmCoeff
 * (layers.py:341-356) and count_vertex_adjface (decimate_gpu.cu:813-836): about 60 small torch and
 * CUDA kernels in the reference. */
int pb200_level_prepare(int64_t Nf, int64_t NvIn, int64_t NvOut, int vstride, const float* vertex,
                        const int32_t* face, const int32_t* vtMap, int L, int orient,
                        float* geometry, float* normals, float* coeff, int32_t* nfCount,
                        int32_t* rowptr, int32_t* entries, int32_t* status,
                        void* workspace, size_t workspace_bytes, void* stream);

/* ---- mesh pooling / unpooling over decimation clusters ------------------------------------
 * Cluster encoding of the fine level (picasso/mesh/pi_modules/decimate.py:23-28): vtReplace[v] < 0
 * names the representative -vtReplace[v] that v was contracted into; a representative holds its
 * cluster size minus one; vtMap[representative] is the coarse vertex id, vtMap of every other
 * vertex is -1.
 *
 * pb200_build_cluster_csr turns the encoding into the two structures the kernels pull through:
 * key[v] = coarse id of the cluster of fine vertex v (or -1), and a CSR coarse vertex -> member
 * fine vertices in ascending order (rowptr NvOut+1 ints, members NvIn ints).  `status` is set to 0
 * or PB200_EINDEX (a representative outside [0,NvIn) or a vtMap value outside [-1,NvOut); such
 * vertices get key -1 and are never dereferenced).  The reference has no such structure: it
 * scatters with compare-and-swap / float atomics (mesh_pool3d_gpu.cu:6-17,62,130; mesh_unpool3d_gpu.cu:43). */
size_t pb200_cluster_csr_workspace_bytes(int64_t NvIn, int64_t NvOut);
int pb200_build_cluster_csr(int64_t NvIn, int64_t NvOut, const int32_t* vtReplace, const int32_t* vtMap,
                            int32_t* key, int32_t* rowptr, int32_t* members, int32_t* status,
                            void* workspace, size_t workspace_bytes, void* stream);

/* output[vo,c] = max over the members v of cluster vo of input[v,c]; maxIndex[vo,c] = the member that
 * attains it (the smallest id among ties; the reference leaves ties to its thread order).  Replaces
 * maxPool3dLauncher (mesh_pool3d_gpu.cu:20-88,162-169; binding mesh_pool3d.cpp MeshMaxPool3d).
 * input (NvIn,C), output (NvOut,C), maxIndex (NvOut,C) int32. */
int pb200_mesh_max_pool_forward(int64_t NvIn, int64_t NvOut, int C, const float* input, const int32_t* rowptr,
                                const int32_t* members, float* output, int32_t* maxIndex, void* stream);
/* gradInput = 0 except gradInput[maxIndex[vo,c], c] = gradOutput[vo,c].  Replaces maxPool3dGradLauncher
 * (mesh_pool3d_gpu.cu:93-105,171-177; binding MeshMaxPool3dGrad). */
int pb200_mesh_max_pool_backward(int64_t NvIn, int64_t NvOut, int C, const int32_t* maxIndex, const float* gradOutput,
                                 float* gradInput, void* stream);
/* The same gradient for a caller that holds the cluster structures of pb200_build_cluster_csr (key, rowptr) and a
 * maxIndex made by pb200_mesh_max_pool_forward over them: every row of gradInput is written once by a gather
 * (row v takes gradOutput[key[v],c] where maxIndex[key[v],c] == v), no zero fill and no scattered stores; identical
 * result, members-less coarse vertices included (their gradient goes to vertex 0 as in the scatter). */
int pb200_mesh_max_pool_backward_clusters(int64_t NvIn, int64_t NvOut, int C, const int32_t* maxIndex,
                                          const float* gradOutput, const int32_t* key, const int32_t* rowptr,
                                          float* gradInput, void* stream);
/* output[vo,c] = sum over members of input[v,c] / (vtReplace[representative] + 1).  Replaces
 * avgPool3dLauncher (mesh_pool3d_gpu.cu:112-132,179-185; binding MeshAvgPool3d). */
int pb200_mesh_avg_pool_forward(int64_t NvIn, int64_t NvOut, int C, const float* input, const int32_t* vtReplace,
                                const int32_t* rowptr, const int32_t* members, float* output, void* stream);
/* gradInput[v,c] = gradOutput[key[v],c] / count for cluster members, 0 elsewhere.  Replaces
 * avgPool3dGradLauncher (mesh_pool3d_gpu.cu:138-158,187-193; binding MeshAvgPool3dGrad). */
int pb200_mesh_avg_pool_backward(int64_t NvIn, int64_t NvOut, int C, const float* gradOutput, const int32_t* vtReplace,
                                 const int32_t* key, float* gradInput, void* stream);
/* Interpolation coarse -> fine: output[v,c] = input[key[v],c] for every fine vertex of a cluster, 0
 * elsewhere; key / rowptr / members are the fine level's cluster structures.  Replaces
 * interpolateLauncher (mesh_unpool3d_gpu.cu:5-26,49-55; binding mesh_unpool3d.cpp MeshInterpolate). */
int pb200_mesh_unpool_forward(int64_t NvCoarse, int64_t NvFine, int C, const float* input, const int32_t* key,
                              float* output, void* stream);
/* gradInput[vo,c] = sum over the members v of cluster vo of gradOutput[v,c], ascending v.  Replaces
 * interpolateGradLauncher (mesh_unpool3d_gpu.cu:29-46,57-63; binding MeshInterpolateGrad). */
int pb200_mesh_unpool_backward(int64_t NvCoarse, int64_t NvFine, int C, const float* gradOutput, const int32_t* rowptr,
                               const int32_t* members, float* gradInput, void* stream);

/* ---- point-cloud depthwise convolution (the SPH3D kernel of the dual point / mesh blocks) ------
 * Neighbour pairs p = (nnIndex[p][0] = output point, nnIndex[p][1] = input point), Nout of them;
 * nnCount[o] = neighbours of output point o; a pair's filter bin is binIndex[p] (hard assignment,
 * binCoeff = NULL, T = 1) or the T bins binIndex[p][t] with weights binCoeff[p][t] (fuzzy).
 *   output[o, c*r+m] = sum over the pairs of o of input[in_p, c] * w_p[c*r+m] / nnCount[o],
 *   w_p[co] = filter[bin_p, co]  or  sum_t binCoeff[p][t] * filter[binIndex[p][t], co].
 * Replaces depthwiseConv3dLauncher / fuzzyDepthwiseConv3dLauncher and their Grad launchers
 * (picasso/point/pi_modules/source/pcloud_conv3d_gpu.cu:8-193,197-268; bindings pcloud_conv3d.cpp
 * SPH3D_forward/backward, fuzzySPH3D_forward/backward).  input (Np,C), filter (F,C,r), output (Mp,C*r).
 * The pairs are pulled through two groupings built with pb200_build_key_csr: by output point
 * (key = nnIndex, stride 2) for the forward pass, by input point (key = nnIndex + 1, stride 2) for the
 * input gradient.  Indices outside their range contribute nothing. */

/* Generic grouping of N items by key[i * key_stride] in [-1, NvOut): rowptr (NvOut+1), members (N)
 * = item ids of every row in ascending order; `status` = 0 or PB200_EINDEX.  Workspace as
 * pb200_cluster_csr_workspace_bytes(N, NvOut). */
int pb200_build_key_csr(int64_t N, int64_t NvOut, const int32_t* key, int key_stride, int32_t* rowptr,
                        int32_t* members, int32_t* status, void* workspace, size_t workspace_bytes, void* stream);
int pb200_pcloud_conv3d_forward(int64_t Np, int64_t Mp, int64_t Nout, int F, int C, int r, int T,
                                const float* input, const float* filter, const int32_t* nnCount,
                                const int32_t* nnIndex, const int32_t* binIndex, const float* binCoeff,
                                const int32_t* rowptr_out, const int32_t* members_out, float* output, void* stream);
size_t pb200_pcloud_conv3d_backward_workspace_bytes(int64_t Nout, int F, int C, int r);
int pb200_pcloud_conv3d_backward(int64_t Np, int64_t Mp, int64_t Nout, int F, int C, int r, int T,
                                 const float* gradOutput, const float* input, const float* filter,
                                 const int32_t* nnCount, const int32_t* nnIndex, const int32_t* binIndex,
                                 const float* binCoeff, const int32_t* rowptr_in, const int32_t* members_in,
                                 float* gradInput, float* gradFilter, void* workspace, size_t workspace_bytes,
                                 void* stream);

/* ---- mesh decimation (one pass) and cluster merge ----------------------------------------
 * pb200_mesh_simplify replaces meshDecimationLauncher (picasso/mesh/pi_modules/source/decimate_gpu.cu:618-747;
 * binding decimate.cpp MeshDecimation, Python module function `simplify`): one pass of quadric-error vertex
 * clustering over a batch of B meshes.  nvIn / mfIn (B) are the running totals of vertices / faces per sample
 * (the last ones equal Nv / Nf), nv2Remove (B) the vertices to remove per sample; vertexIn (Nv,D>=3),
 * faceIn (Nf,3), planeIn (Nf,5) = unit normal, plane intercept, area.  Outputs as the reference's:
 * vertexOut (Nv,D) (cluster means; zero rows for contracted vertices), faceOut (Nf,3) (relabelled to output
 * ids where not degenerate), isDegenerate (Nf) bytes, vtReplace (Nv) (negative = contracted into that vertex,
 * positive = cluster size - 1, 0 = untouched), vtMap (Nv) (output id or -1), nvOut / mfOut (B).
 * Everything runs on the device; the reference's per-sample host loop and its sequential clustering sweeps
 * (decimate_gpu.cu:561-614) are computed as parallel rounds with the same result.  Where the reference adds
 * floats with atomics, the order here is fixed: quadrics by ascending (face, corner), cluster means by
 * ascending vertex id, and no multiply-add is fused, so the result is reproducible bit for bit.  Candidates
 * with equal cost keep their (lower vertex, higher vertex) order; -0 counts as +0, NaN costs come last.
 * Edges of a face that names a vertex twice are no candidates.
 * edgeCost (3*Nf floats, may be NULL) receives the cost of every distinct edge in (lower, higher) order;
 * info (HOST pointer to 4 int64, may be NULL) = {distinct edges, matching rounds run on the whole grid, edges
 * handed to the single-block finish, 0}.  The call synchronises the stream a few times (it reads back three
 * counters and the 2*B sample totals) and returns PB200_EINDEX for a vertex id outside [0, Nv). */
size_t pb200_mesh_simplify_workspace_bytes(int64_t B, int64_t Nv, int64_t Nf);
int pb200_mesh_simplify(int useArea, float wgtBnd, int64_t B, int64_t D, int64_t Nv, int64_t Nf,
                        const int32_t* nvIn, const int32_t* mfIn, const int32_t* nv2Remove, const float* vertexIn,
                        const int32_t* faceIn, const float* planeIn, int32_t* nvOut, int32_t* mfOut, float* vertexOut,
                        int32_t* faceOut, int32_t* vtReplace, int32_t* vtMap, uint8_t* isDegenerate, float* edgeCost,
                        int64_t* info, void* workspace, size_t workspace_bytes, void* stream);
/* Clusters of a mesh A (repA, mapA over its nvA vertices) merged with the clusters of its decimated
 * version B (repB, mapB over nvB vertices) into clusters of A over the vertices B kept.  Replaces
 * combineClustersLauncher (decimate_gpu.cu:750-812; binding CombineClusters, `combine_clusters`).
 * Workspace: (nvB + 1) int32; `status` = 0 or PB200_EINDEX (an id out of range, skipped). */
int pb200_combine_clusters(int64_t nvA, int64_t nvB, const int32_t* repA, const int32_t* mapA, const int32_t* repB,
                           const int32_t* mapB, int32_t* repOut, int32_t* mapOut, int32_t* status, void* workspace,
                           size_t workspace_bytes, void* stream);

/* ---- row expansion (benchmark block glue) ----------------------------------------------
 * forward:  out[k,:] = in[f,:] for every sample k of face f (numInterior as above);
 * backward: gradIn[f,:] = sum over the samples k of f of gradOut[k,:] (fixed order).
 * The reference does this with torch.repeat_interleave in user code; there is no
 * counterpart inside its extension. */
int pb200_expand_rows_forward(int64_t Nf, int64_t NiK, int C, const float* in, const int32_t* numInterior,
                              float* out, void* stream);
int pb200_expand_rows_backward(int64_t Nf, int64_t NiK, int C, const float* gradOut, const int32_t* numInterior,
                               float* gradIn, void* stream);

/* out[f,:] = mean over the samples k of face f of rows[k,:], added in ascending order; 0 for a face without
 * samples.  With one input row per face shared by all its samples (the block's repeat_interleave followed by
 * facet2facet), the face operand of facet2facet factorises:
 *   (1/T_f) sum_k bary[k,d] * in[f,ci] = mean_k(bary[k,d]) * in[f,ci],
 * so facet2facet over (in (Nf,Cin), mean rows (Nf,F), numInterior = 1, 2, ..., Nf) gives the same output and the
 * same gradients as the expanded call (the input gradient already summed per face), without the expanded rows.
 * No counterpart inside the reference's extension. */
int pb200_face_mean_rows(int64_t Nf, int64_t NiK, int C, const float* rows, const int32_t* numInterior, float* out,
                         void* stream);
/* The same per-face mean for rows that are the spherical-harmonic components of sample positions: out[f,:] =
 * mean over the samples k of face f of pb200_sph_harm_coeff(xyz[k]) (identical bits), without the (NiK,(L+1)^2) array
 * in between.  xyz (NiK,3), out (Nf,(L+1)^2), L <= 5. */
int pb200_face_mean_sph_harm(int64_t Nf, int64_t NiK, int L, const float* xyz, const int32_t* numInterior, float* out,
                             void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PICASSO_B200_H */
