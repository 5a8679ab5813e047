/* A C (not C++) translation unit that includes the library's header and calls its host-only entry points:
 * the header must be valid C and the shared library must link against a plain C program, as a cgo / JNI /
 * ctypes binding of the operator surface would require. */
#include <stdio.h>
#include <string.h>

#include "kvcomp_b200.h"

int main(void) {
    int64_t out[4];
    kvc_qmeta q;
    int64_t units = 0;
    if (kvc_version() != KVC_VERSION) return 1;
    if (kvc_buffer_sizes(1024, 32 * 128, 1, out) != KVC_OK || out[0] != 4096 || out[1] != 65536 || out[3] != 4194304) return 2;
    if (kvc_buffer_sizes(1000, 32 * 128, 1, out) != KVC_ERR_ARG || strlen(kvc_last_error()) == 0) return 3;
    memset(&q, 0, sizeof q);
    if (kvc_qmeta_make(KVC_MODE_CHANNEL, 0, 128, 2, 4, 128, 64, &q, &units) != KVC_OK || units != 2 * 2 * 4 * 128 || q.sc != 1) return 4;
    if (kvc_attn_workspace(8, 32, 8) != 256 + 8 * 32 * 8 * 260 * 4) return 5;
    if (kvc_attn_decode(NULL, NULL, 128, 1, 1, 1, NULL, 1.0f, NULL, NULL, 0, NULL, 0, NULL, 0, NULL, NULL) != KVC_ERR_ARG) return 6;
    printf("ok %d %d %d\n", KVC_BOOK_BYTES, (int)sizeof(kvc_cache), (int)sizeof(kvc_qmeta));   /* the caller compares with its ctypes structures */
    return 0;
}
