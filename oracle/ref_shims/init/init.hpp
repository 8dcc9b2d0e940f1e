// Stand-in for the reference's init/init.hpp (logger, flags, cuBLAS handle):
// its kernel headers include it but use nothing from it.
#pragma once
