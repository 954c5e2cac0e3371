/* C API of the inference engine: the five entry points of the reference's extern "C" block
 * (include/oil/production.h:134-141), exported by liboil_capi.so for programs in any language that can call C.
 *
 * The engine behind the handle is this package's Python / PyTorch generator: the library starts (or joins) a Python
 * interpreter in the calling process. Which interpreter: the executable named by INNOVA_B200_PYTHON, else "python3" on
 * PATH (a virtual environment's python brings its site-packages with it). Where the package is: INNOVA_B200_ROOT, else
 * the directory two levels above this library. Calls may come from any thread; they are serialised by the
 * interpreter lock. No call throws; a failed call returns NULL and oil_last_error() (per thread) says why.
 */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

typedef struct OilModel OilModel;

OilModel* oil_model_load(const char* path);                                   /* NULL on failure */
void oil_model_free(OilModel* model);                                         /* NULL is accepted */
char* oil_generate(OilModel* model, const char* prompt, int max_tokens);      /* malloc'd UTF-8 text, NULL on failure */
void oil_free_string(char* s);                                                /* for strings returned by oil_generate */
const char* oil_last_error(void);                                             /* "" when the last call on this thread succeeded */

#ifdef __cplusplus
}
#endif
