// fp16 build of step.cu (namespace clt_h, C symbols with the suffix _h)
#define CLT_HALF 1
#include "../step.cu"
