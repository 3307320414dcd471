// Stand-in for the one library header that rocWMMA's CPU reference file includes
// but whose contents the GEMM / DLRM host functions never use.  Found through
// -I when the reference's own sources are compiled into oracle/_ref (see the
// Makefile); it keeps that build free of HIP.
#pragma once
