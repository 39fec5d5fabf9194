/*
 * Minimal stand-in for MATLAB's mex.h, for syntax-checking the MEX gateway
 * (nnv_b200/csrc/nnvb200_mex.cpp) on machines without MATLAB.  It declares only
 * the documented MEX/MX API functions the gateway calls, with the documented
 * signatures.  It is never linked: a real build uses MATLAB's own header via
 * `mex`.
 */
#ifndef NNVB_MEX_STUB_H
#define NNVB_MEX_STUB_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
typedef struct mxArray_tag mxArray;
typedef size_t mwSize;
typedef size_t mwIndex;
typedef enum { mxUNKNOWN_CLASS = 0, mxDOUBLE_CLASS = 6, mxINT32_CLASS = 12, mxUINT64_CLASS = 15 } mxClassID;
typedef enum { mxREAL = 0, mxCOMPLEX = 1 } mxComplexity;
typedef double mxDouble;
typedef uint64_t mxUint64;
bool mxIsDouble(const mxArray*);
bool mxIsChar(const mxArray*);
bool mxIsStruct(const mxArray*);
bool mxIsCell(const mxArray*);
bool mxIsEmpty(const mxArray*);
bool mxIsComplex(const mxArray*);
mxDouble* mxGetDoubles(const mxArray*);
void* mxGetData(const mxArray*);
double mxGetScalar(const mxArray*);
mwSize mxGetNumberOfDimensions(const mxArray*);
const mwSize* mxGetDimensions(const mxArray*);
size_t mxGetNumberOfElements(const mxArray*);
size_t mxGetM(const mxArray*);
size_t mxGetN(const mxArray*);
mxArray* mxGetField(const mxArray*, mwIndex, const char*);
mxArray* mxGetCell(const mxArray*, mwIndex);
char* mxArrayToString(const mxArray*);
void mxFree(void*);
mxArray* mxCreateNumericArray(mwSize ndim, const mwSize* dims, mxClassID, mxComplexity);
mxArray* mxCreateNumericMatrix(mwSize m, mwSize n, mxClassID, mxComplexity);
mxArray* mxCreateDoubleMatrix(mwSize m, mwSize n, mxComplexity);
mxArray* mxCreateDoubleScalar(double);
mxArray* mxCreateStructMatrix(mwSize m, mwSize n, int nfields, const char** fieldnames);
void mxSetField(mxArray*, mwIndex, const char*, mxArray*);
void mexErrMsgIdAndTxt(const char* id, const char* fmt, ...);
void mexLock(void);
void mexUnlock(void);
int mexAtExit(void (*fn)(void));
#ifdef __cplusplus
}
#endif
#endif
