// fp16 build of theta_grad_gemm.cu (namespace clt_h, C symbols with the suffix _h)
#define CLT_HALF 1
#include "../theta_grad_gemm.cu"
