/* Status and error helpers with the reference's behaviour
 * (include/yvex/core.h:28-48, src/core/status.c). */
#include "private.h"

#include <stdio.h>
#include <string.h>

void yvex_error_clear(yvex_error *err)
{
    if (!err) return;
    err->code = YVEX_OK;
    err->where[0] = '\0';
    err->message[0] = '\0';
}

void yvex_error_set(yvex_error *err, yvex_status code, const char *where, const char *message)
{
    if (!err) return;
    err->code = code;
    snprintf(err->where, sizeof(err->where), "%s", where ? where : "");
    snprintf(err->message, sizeof(err->message), "%s", message ? message : "");
}

const char *yvex_status_name(yvex_status status)
{
    switch (status) {
    case YVEX_OK: return "ok";
    case YVEX_ERR: return "error";
    case YVEX_ERR_NOMEM: return "nomem";
    case YVEX_ERR_IO: return "io";
    case YVEX_ERR_FORMAT: return "format";
    case YVEX_ERR_UNSUPPORTED: return "unsupported";
    case YVEX_ERR_BACKEND: return "backend";
    case YVEX_ERR_BOUNDS: return "bounds";
    case YVEX_ERR_STATE: return "state";
    case YVEX_ERR_CANCELLED: return "cancelled";
    case YVEX_ERR_INVALID_ARG: return "invalid-arg";
    case YVEX_ERR_TIMEOUT: return "timeout";
    }
    return "unknown";
}

int yvx_fail(yvex_error *err, yvex_status code, const char *where, const char *message)
{
    yvex_error_set(err, code, where, message);
    return (int)code;
}

unsigned long long yvx_dtype_bytes(yvex_dtype dtype)
{
    switch (dtype) {
    case YVEX_DTYPE_F32: case YVEX_DTYPE_I32: return 4ull;
    case YVEX_DTYPE_F16: case YVEX_DTYPE_BF16: case YVEX_DTYPE_I16: return 2ull;
    case YVEX_DTYPE_F64: case YVEX_DTYPE_I64: return 8ull;
    case YVEX_DTYPE_I8: return 1ull;
    default: return 0ull;
    }
}
