// elementwise_rows_outer.cu -- the instantiations of rows_kernel that carry an outer index (broadcasts over three
// axes), in a translation unit of their own so that they compile beside the rest of elementwise_impl.cuh.
#define BSIR_ELEMENTWISE_PART_OUTER 1
#include "elementwise_impl.cuh"
