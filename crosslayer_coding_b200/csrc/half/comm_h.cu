// fp16 build of comm.cu (namespace clt_h, C symbols with the suffix _h)
#define CLT_HALF 1
#include "../comm.cu"
