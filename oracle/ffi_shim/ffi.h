/* Minimal declarations of the public libffi API (x86-64 System V) for linking
 * against the system's libffi.so.8 when its development headers are not
 * installed.  Only the names the GeNN runtime uses are declared.  This is test
 * infrastructure for building the CPU reference; the product does not use it. */
#ifndef ORACLE_FFI_SHIM_H
#define ORACLE_FFI_SHIM_H
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef struct _ffi_type {
    size_t size;
    unsigned short alignment;
    unsigned short type;
    struct _ffi_type **elements;
} ffi_type;

typedef enum { FFI_OK = 0, FFI_BAD_TYPEDEF, FFI_BAD_ABI, FFI_BAD_ARGTYPE } ffi_status;

typedef enum ffi_abi {
    FFI_FIRST_ABI = 1,
    FFI_UNIX64,
    FFI_WIN64,
    FFI_EFI64 = FFI_WIN64,
    FFI_GNUW64,
    FFI_LAST_ABI,
    FFI_DEFAULT_ABI = FFI_UNIX64
} ffi_abi;

typedef struct {
    ffi_abi abi;
    unsigned nargs;
    ffi_type **arg_types;
    ffi_type *rtype;
    unsigned bytes;
    unsigned flags;
} ffi_cif;

extern ffi_type ffi_type_void;
extern ffi_type ffi_type_uint8, ffi_type_sint8;
extern ffi_type ffi_type_uint16, ffi_type_sint16;
extern ffi_type ffi_type_uint32, ffi_type_sint32;
extern ffi_type ffi_type_uint64, ffi_type_sint64;
extern ffi_type ffi_type_float, ffi_type_double, ffi_type_pointer;

#define ffi_type_uint ffi_type_uint32
#define ffi_type_sint ffi_type_sint32
#define FFI_FN(f) ((void (*)(void))f)

ffi_status ffi_prep_cif(ffi_cif *cif, ffi_abi abi, unsigned int nargs,
                        ffi_type *rtype, ffi_type **atypes);
void ffi_call(ffi_cif *cif, void (*fn)(void), void *rvalue, void **avalue);

#ifdef __cplusplus
}
#endif
#endif
