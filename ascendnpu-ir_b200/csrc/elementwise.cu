// elementwise.cu -- hfusion.elemwise_unary / elemwise_binary / compare / select, copies, and the C entry points for
// them: the main part of elementwise_impl.cuh.
#include "elementwise_impl.cuh"
