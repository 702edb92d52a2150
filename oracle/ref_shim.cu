// ref_shim.cu -- builds the reference's own CUDA translation unit (CudaStuff.cu) into a shared
// library that GPU parity tests load beside the oracle.  TEST INFRASTRUCTURE ONLY.
//
// The reference source is compiled from where it lies (the include path is supplied by the
// Makefile: -I"<reference>/AI gamer"); nothing of it is copied here.  This file only adds what the
// reference's Windows-only common.cpp would have supplied at link time, plus a launcher that runs
// the reference's own LayerNorm kernels with one block per channel, which is what the statistics
// kernel expects (it indexes channels by blockIdx.x, CudaStuff.cu:460) while the reference launcher
// starts only ceil(C/BS) blocks (CudaStuff.cu:509).
#include "CudaStuff.cu"

// common.cpp:48-85 maps a compute capability to "cores per SM" and the launchers use it as their
// block size BS.  The table there stops before sm_100, so the value is fixed to the one the
// reference was built for (sm_70 -> 64).
int ConvertSmVer2Cores(int, int) { return 64; }

extern "C" void ref_set_launch_shape(int gs, int bs) {
  GS = gs;
  BS = bs;
}
extern "C" int ref_get_bs() { return BS; }

extern "C" int ref_layernorm_forward_fullgrid(__half* output, const __half* data, const float* gamma,
                                              const float* beta, float* mean, float* variance, int N,
                                              int C, int HW) {
  ComputeMeanVarianceKernel<<<C, BS, 3 * BS * sizeof(float)>>>(data, mean, variance, N, C, HW);
  int gridSize = div_ceil(N * C * HW, BS);
  layerNormForwardKernel<<<gridSize, BS, 4 * C * sizeof(float)>>>(output, data, gamma, beta, mean,
                                                                  variance, N, C, HW);
  return (int)cudaGetLastError();
}
