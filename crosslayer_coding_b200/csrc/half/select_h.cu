// fp16 build of select.cu (namespace clt_h, C symbols with the suffix _h)
#define CLT_HALF 1
#include "../select.cu"
