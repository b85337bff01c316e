// Same name as lutGEMM/include/kernels.h of the reference; the functions live in lutgemm_compat.hpp.
#include "lutgemm_compat.hpp"
