// Forwarding header: the drop-in declarations for this reference header live in lh_dropin.hpp.
#include "../lh_dropin.hpp"
