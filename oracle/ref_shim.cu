// C-ABI doorway to the reference's own host launchers, so that the parity tests can call
// the unmodified reference CUDA kernels through ctypes.  TEST INFRASTRUCTURE ONLY.
// This file holds declarations and forwarding calls only; the kernels themselves are
// compiled from the reference tree where it lies (see oracle/Makefile, target `ref`).
// Launcher signatures: picasso/mesh/pi_modules/source/mesh_conv3d.cpp:9-23,
// picasso/mesh/pi_modules/source/decimate.cpp:9-17 (meshDecimationLauncher, combineClustersLauncher,
// countVertexAdjfaceLauncher),
// mesh_pool3d.cpp:8-15, mesh_unpool3d.cpp:8-11 and picasso/point/pi_modules/source/pcloud_conv3d.cpp:8-21.
#include <cuda_runtime.h>

void facet2vertexConv3dLauncher(int NfIn, int C, int r, int K, const int* vtMap, const int* nfCount, const int* face,
                                const float* coeff, const float* input, const float* filter, float* output);
void vertex2facetConv3dLauncher(int NfIn, int C, int r, const int* face,
                                const float* input, const float* filter, float* output);
void facet2facetConv3dLauncher(int NfIn, int F, int Cin, int Cout, const int* numInterior, const float* intrplWgts,
                               const float* input, const float* filter, float* output);
void facet2vertexConv3dGradLauncher(int NfIn, int C, int r, int K, const int* vtMap, const int* nfCount, const int* face,
                                    const float* coeff, const float* input, const float* filter, const float* gradOutput,
                                    float* gradInput, float* gradFilter);
void vertex2facetConv3dGradLauncher(int NfIn, int C, int r, const int* face, const float* input, const float* filter,
                                    const float* gradOutput, float* gradInput, float* gradFilter);
void facet2facetConv3dGradLauncher(int NfIn, int F, int Cin, int Cout, const int* numInterior, const float* intrplWgts,
                                   const float* input, const float* filter, const float* gradOutput,
                                   float* gradInput, float* gradFilter);
void countVertexAdjfaceLauncher(int NfIn, const int* face, const int* vtMap, int* nfCount);
void meshDecimationLauncher(const bool useArea, const float wgtBnd, const int B, const int D, const int Nv, const int Nf,
                            const int* nvIn, const int* mfIn, const int* nv2Remove, const float* vertexIn,
                            const int* faceIn, const float* planeIn, int* nvOut, int* mfOut, float* vertexOut,
                            int* faceOut, int* vtReplace, int* vtMap, bool* isDegenerate);
void combineClustersLauncher(const int nvA, const int nvB, const int* repA, const int* mapA, const int* repB,
                             const int* mapB, int* repOut, int* mapOut);
void maxPool3dLauncher(int nvIn, int C, const int* vtReplace, const int* vtMap, const float* input, float* output,
                       int* maxIndex);
void maxPool3dGradLauncher(int nvOut, int C, const int* maxIndex, const float* gradOutput, float* gradInput);
void avgPool3dLauncher(int nvIn, int C, const int* vtReplace, const int* vtMap, const float* input, float* output);
void avgPool3dGradLauncher(int nvIn, int C, const int* vtReplace, const int* vtMap, const float* gradOutput,
                           float* gradInput);
void interpolateLauncher(int nvIn, int C, int nvOut, const int* vtReplace, const int* vtMap, const float* input,
                         float* output);
void interpolateGradLauncher(int nvIn, int C, int nvOut, const int* vtReplace, const int* vtMap, const float* gradOutput,
                             float* gradInput);
void depthwiseConv3dLauncher(int Np, int Mp, int Nout, int F, int C, int r, const int* nnCount, const int* nnIndex,
                             const int* binIndex, const float* input, const float* filter, float* output);
void depthwiseConv3dGradLauncher(int Np, int Mp, int Nout, int F, int C, int r, const int* nnCount, const int* nnIndex,
                                 const int* binIndex, const float* input, const float* filter, const float* gradOutput,
                                 float* gradInput, float* gradFilter);
void fuzzyDepthwiseConv3dLauncher(int Np, int Mp, int Nout, int F, int C, int r, int T, const int* nnCount,
                                  const int* nnIndex, const int* binIndex, const float* binCoeff, const float* input,
                                  const float* filter, float* output);
void fuzzyDepthwiseConv3dGradLauncher(int Np, int Mp, int Nout, int F, int C, int r, int T, const int* nnCount,
                                      const int* nnIndex, const int* binIndex, const float* binCoeff, const float* input,
                                      const float* filter, const float* gradOutput, float* gradInput, float* gradFilter);

// The reference launches on the legacy default stream and never checks errors; each
// doorway synchronises the device and returns the CUDA status so a test can assert on it.
static int finish() {
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaGetLastError();
    return (int)e;
}

extern "C" {
int ref_f2v_forward(int NfIn, int C, int r, int K, const int* vtMap, const int* nfCount, const int* face,
                    const float* coeff, const float* input, const float* filter, float* output) {
    facet2vertexConv3dLauncher(NfIn, C, r, K, vtMap, nfCount, face, coeff, input, filter, output);
    return finish();
}
int ref_v2f_forward(int NfIn, int C, int r, const int* face, const float* input, const float* filter, float* output) {
    vertex2facetConv3dLauncher(NfIn, C, r, face, input, filter, output);
    return finish();
}
int ref_f2f_forward(int NfIn, int F, int Cin, int Cout, const int* numInterior, const float* bary,
                    const float* input, const float* filter, float* output) {
    facet2facetConv3dLauncher(NfIn, F, Cin, Cout, numInterior, bary, input, filter, output);
    return finish();
}
int ref_f2v_backward(int NfIn, int C, int r, int K, const int* vtMap, const int* nfCount, const int* face,
                     const float* coeff, const float* input, const float* filter, const float* gradOutput,
                     float* gradInput, float* gradFilter) {
    facet2vertexConv3dGradLauncher(NfIn, C, r, K, vtMap, nfCount, face, coeff, input, filter, gradOutput,
                                   gradInput, gradFilter);
    return finish();
}
int ref_v2f_backward(int NfIn, int C, int r, const int* face, const float* input, const float* filter,
                     const float* gradOutput, float* gradInput, float* gradFilter) {
    vertex2facetConv3dGradLauncher(NfIn, C, r, face, input, filter, gradOutput, gradInput, gradFilter);
    return finish();
}
int ref_f2f_backward(int NfIn, int F, int Cin, int Cout, const int* numInterior, const float* bary,
                     const float* input, const float* filter, const float* gradOutput,
                     float* gradInput, float* gradFilter) {
    facet2facetConv3dGradLauncher(NfIn, F, Cin, Cout, numInterior, bary, input, filter, gradOutput,
                                  gradInput, gradFilter);
    return finish();
}
int ref_count_vertex_adjface(int NfIn, const int* face, const int* vtMap, int* nfCount) {
    countVertexAdjfaceLauncher(NfIn, face, vtMap, nfCount);
    return finish();
}
// The reference keeps one int per vertex in an array on the host stack (decimate_gpu.cu:663):
// callers keep Nv small.
int ref_mesh_simplify(int useArea, float wgtBnd, int B, int D, int Nv, int Nf, const int* nvIn, const int* mfIn,
                      const int* nv2Remove, const float* vertexIn, const int* faceIn, const float* planeIn, int* nvOut,
                      int* mfOut, float* vertexOut, int* faceOut, int* vtReplace, int* vtMap, bool* isDegenerate) {
    meshDecimationLauncher(useArea != 0, wgtBnd, B, D, Nv, Nf, nvIn, mfIn, nv2Remove, vertexIn, faceIn, planeIn, nvOut,
                           mfOut, vertexOut, faceOut, vtReplace, vtMap, isDegenerate);
    return finish();
}
int ref_combine_clusters(int nvA, int nvB, const int* repA, const int* mapA, const int* repB, const int* mapB,
                         int* repOut, int* mapOut) {
    combineClustersLauncher(nvA, nvB, repA, mapA, repB, mapB, repOut, mapOut);
    return finish();
}
int ref_max_pool_forward(int nvIn, int C, const int* vtReplace, const int* vtMap, const float* input, float* output,
                         int* maxIndex) {
    maxPool3dLauncher(nvIn, C, vtReplace, vtMap, input, output, maxIndex);
    return finish();
}
int ref_max_pool_backward(int nvOut, int C, const int* maxIndex, const float* gradOutput, float* gradInput) {
    maxPool3dGradLauncher(nvOut, C, maxIndex, gradOutput, gradInput);
    return finish();
}
int ref_avg_pool_forward(int nvIn, int C, const int* vtReplace, const int* vtMap, const float* input, float* output) {
    avgPool3dLauncher(nvIn, C, vtReplace, vtMap, input, output);
    return finish();
}
int ref_avg_pool_backward(int nvIn, int C, const int* vtReplace, const int* vtMap, const float* gradOutput,
                          float* gradInput) {
    avgPool3dGradLauncher(nvIn, C, vtReplace, vtMap, gradOutput, gradInput);
    return finish();
}
int ref_unpool_forward(int nvIn, int C, int nvOut, const int* vtReplace, const int* vtMap, const float* input,
                       float* output) {
    interpolateLauncher(nvIn, C, nvOut, vtReplace, vtMap, input, output);
    return finish();
}
int ref_unpool_backward(int nvIn, int C, int nvOut, const int* vtReplace, const int* vtMap, const float* gradOutput,
                        float* gradInput) {
    interpolateGradLauncher(nvIn, C, nvOut, vtReplace, vtMap, gradOutput, gradInput);
    return finish();
}
int ref_pcloud_forward(int Np, int Mp, int Nout, int F, int C, int r, int T, const int* nnCount, const int* nnIndex,
                       const int* binIndex, const float* binCoeff, const float* input, const float* filter, float* output) {
    if (binCoeff) fuzzyDepthwiseConv3dLauncher(Np, Mp, Nout, F, C, r, T, nnCount, nnIndex, binIndex, binCoeff, input, filter, output);
    else depthwiseConv3dLauncher(Np, Mp, Nout, F, C, r, nnCount, nnIndex, binIndex, input, filter, output);
    return finish();
}
int ref_pcloud_backward(int Np, int Mp, int Nout, int F, int C, int r, int T, const int* nnCount, const int* nnIndex,
                        const int* binIndex, const float* binCoeff, const float* input, const float* filter,
                        const float* gradOutput, float* gradInput, float* gradFilter) {
    if (binCoeff)
        fuzzyDepthwiseConv3dGradLauncher(Np, Mp, Nout, F, C, r, T, nnCount, nnIndex, binIndex, binCoeff, input, filter,
                                         gradOutput, gradInput, gradFilter);
    else
        depthwiseConv3dGradLauncher(Np, Mp, Nout, F, C, r, nnCount, nnIndex, binIndex, input, filter, gradOutput, gradInput,
                                    gradFilter);
    return finish();
}
}
