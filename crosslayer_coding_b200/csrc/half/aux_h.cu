// fp16 build of aux.cu (namespace clt_h, C symbols with the suffix _h)
#define CLT_HALF 1
#include "../aux.cu"
