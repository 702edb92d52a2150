/* aig_compat.h -- the forward-path launchers of the reference under their own names and signatures
 * (common.h:104-139, NvDisplayCap.h:68-69), so that reference code that calls them links against
 * libaig_b200.so unchanged.  Each is a thin wrapper over the context API of aig_b200.h on a
 * process-wide context: device = the current CUDA device at the first call (the reference always uses
 * device 0), stream = the legacy default stream, as in the reference (CudaStuff.cu launches without a
 * stream argument).  Errors follow the reference: the launchers return void and report nothing
 * (ARGBtoRGB* return the launch status); the status of the last wrapped call is available through
 * aig_compat_last_status().  Training launchers (optimisers, gradients, losses, backward passes) are
 * not part of the inference path and are not provided. */
#ifndef AIG_COMPAT_H
#define AIG_COMPAT_H
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

void InitCUDA(void);                                                                   /* CudaStuff.cu:20-51 */
void ConvertAndNormalize(__half* output, const unsigned char* input, size_t size);     /* CudaStuff.cu:150-157 */
void UnConvertAndUnNormalize(unsigned char* output, const __half* input, size_t size); /* CudaStuff.cu:158-165 */
void ConvertFloatToHalf(float* src, __half* dst, size_t n);                            /* CudaStuff.cu:166-173 */
void ConvertHalfToFloat(__half* src, float* dst, size_t n);                            /* CudaStuff.cu:174-181 */
void HeInit(__half* weightHalf, int numWeights, float fanIn);                          /* CudaStuff.cu:182-193 */
void LeakyReluForward(__half* data, int size, float negativeSlope);                    /* CudaStuff.cu:400-405 */
void SwishForward(__half* data, int size);                                             /* CudaStuff.cu:416-421 */
void SigmoidForward(__half* data, int numCtrls, int numButs, int size);                /* CudaStuff.cu:437-442 */
void LayerNormForward(__half* output, const __half* data, const float* gamma, const float* beta, float* mean,
                      float* variance, int N, int C, int HW);                          /* CudaStuff.cu:457-515 */
void SpatialAttentionForward(const __half* inData, const __half* keyWeights, const __half* queryWeights,
                             const __half* valueWeights, __half* keyMap, __half* queryMap, __half* valueMap,
                             __half* attentionScores, __half* outData, int batchSize, int inC, int attC, int inH,
                             int inW);                                                 /* CudaStuff.cu:673-760 */
cudaError_t ARGBtoRGB(unsigned char* src, unsigned char* dst, int n);                  /* CudaStuff.cu:52-62 */
cudaError_t ARGBtoRGBplanar(unsigned char* src, unsigned char* dst, int n);            /* CudaStuff.cu:63-74 */
/* training step (see aig_b200.h: losses, gradient, NaN check, activation backward, optimisers) */
float MseLoss(const __half* dPredictions, const float* dTargets, int size);            /* CudaStuff.cu:97-105 */
void MseLoss2(const __half* dPredictions, const float* dTargets, int numButs, int numCtrls, int batchSize, float* butLoss,
              float* axesLoss);                                                        /* CudaStuff.cu:138-151 */
void Gradient(__half* dGradient, const __half* dPredictions, const __half* dTargets, int size);   /* CudaStuff.cu:304-307 */
bool IsnanHalf(const __half* data, int size);                                          /* CudaStuff.cu:576-583 */
void LeakyReluBackward(__half* grad, const __half* data, int size, float negativeSlope);          /* CudaStuff.cu:412-415 */
void SwishBackward(__half* grad, const __half* data, int size);                        /* CudaStuff.cu:433-436 */
void SigmoidBackward(__half* grad, const __half* data, int numCtrls, int numButs, int size);      /* CudaStuff.cu:453-456 */
void BiasGradient(const __half* gradInput, __half* gradBias, int c, int batchSize);    /* CudaStuff.cu:396-399 */
void SGDHalf(__half* params, const __half* grads, int size, float learningRate, float weightDecay);           /* CudaStuff.cu:207-210 */
void SGDFloat(float* params, const float* grads, int size, float learningRate, float weightDecay);            /* CudaStuff.cu:219-222 */
void AdamWFloat(float* params, const float* grads, float* m, float* v, float learningRate, int t, float weightDecay, int size);   /* CudaStuff.cu:233-236 */
void AdamWHalf(__half* params, const __half* grads, __half* m, __half* v, float lr, int t, float weightDecay, int size);          /* CudaStuff.cu:249-252 */

/* Not in the reference: the context behind these wrappers (for mixing them with aig_* calls), the
 * status of the last wrapped call (AIG_OK or a negative code), and the pixel-group size that
 * SpatialAttentionForward derives from the reference's launch block size (default 64). */
struct aig_ctx;
struct aig_ctx* aig_compat_context(void);
int aig_compat_last_status(void);
void aig_compat_set_attention_group(int group);

#ifdef __cplusplus
}
#endif
#endif /* AIG_COMPAT_H */
