// Empty stand-in for <fftw3.h>: the reciprocal-space engine is replaced by no-ops in the oracle build.
#ifndef DSMD_ORACLE_STUB_FFTW3_H
#define DSMD_ORACLE_STUB_FFTW3_H
typedef double fftw_complex[2];
typedef struct dsmd_stub_fftw_plan_s* fftw_plan;
#endif
