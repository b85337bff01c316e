// Same name as lutGEMM/include/nQWeight_fp16.h of the reference; the class lives in lutgemm_compat.hpp.
#include "lutgemm_compat.hpp"
