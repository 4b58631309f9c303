// Forwarding header: the drop-in declarations for this reference header live in lh_dropin.hpp
// (only the functions of the decode step: rmsnorm, rope, swiglu).
#include "../lh_dropin.hpp"
