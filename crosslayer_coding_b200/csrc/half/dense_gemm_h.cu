// fp16 build of dense_gemm.cu (namespace clt_h, C symbols with the suffix _h)
#define CLT_HALF 1
#include "../dense_gemm.cu"
