/* A model's GGUF files as data: their metadata and where each tensor's bytes lie. Nothing past the headers is read or
 * mapped: the weights stay in their files for whoever loads them onto a GPU (tensor t: `bytes` bytes at `offset` of
 * file `paths[t->file]`, ready for quant_dequant / mv_run / mm_run / q8_* by its `type`).
 *
 * Drop-in for the reference's include/osmos/model/gguf.h:42-51 (src/model/gguf.c:49-190): the same structures, the
 * same seven entry points with the same meaning, refusals and ownership.
 *
 * The files are untrusted. Every count, length and offset is checked against the file's size before it is believed or
 * allocated for; a string or array that runs past the end, a tensor whose bytes leave its file, an unknown tensor
 * type, a value count that is not whole blocks, a duplicate tensor name, or a shard that is missing refuses the whole
 * model: NULL, the reason (file, offset, what) in `err`, everything allocated on the way released.
 */
#ifndef OSMOS_B200_GGUF_H
#define OSMOS_B200_GGUF_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GGUF_ERR 256
#define GGUF_MAX_DIMS 4

typedef enum GgufValueType
{
  GGUF_UINT8 = 0,
  GGUF_INT8 = 1,
  GGUF_UINT16 = 2,
  GGUF_INT16 = 3,
  GGUF_UINT32 = 4,
  GGUF_INT32 = 5,
  GGUF_FLOAT32 = 6,
  GGUF_BOOL = 7,
  GGUF_STRING = 8,
  GGUF_ARRAY = 9,
  GGUF_UINT64 = 10,
  GGUF_INT64 = 11,
  GGUF_FLOAT64 = 12
} GgufValueType;

/* One metadata entry. Scalars widened into v.u / v.i / v.f (unsigned and bool, signed, floating); v.s a string (NUL
   terminated, its own copy). An array: `item` its element type, `n` its length, v.items a copy - for strings a
   char ** of n, else n packed values of the element's own width. */
typedef struct GgufKv
{
  char *key;
  GgufValueType type;
  GgufValueType item;
  uint64_t n;
  union
  {
    uint64_t u;
    int64_t i;
    double f;
    char *s;
    void *items;
  } v;
} GgufKv;

/* `type` the ggml type id (qtype.h; also I32 26, I64 27, and 0x12B for a type-43 tensor stored a byte a value),
   `dims` innermost first as in the file, `file` its shard, `offset` its first byte's absolute offset in that file,
   `bytes` its size from its type and dims. */
typedef struct GgufTensor
{
  char *name;
  uint32_t type;
  uint32_t n_dims;
  uint64_t dims[GGUF_MAX_DIMS];
  int file;
  uint64_t offset;
  uint64_t bytes;
} GgufTensor;

/* A split model (`-00001-of-0000N.gguf`) is one Gguf over all its shards: `paths` in shard order, `sizes` each
   file's bytes; the metadata is the first shard's. */
typedef struct Gguf
{
  int n_files;
  char **paths;
  uint64_t *sizes;
  GgufKv *kv;
  size_t n_kv;
  GgufTensor *tensors;
  size_t n_tensors;
} Gguf;

/* `path`: a file, or a split model's first shard (its siblings are found by name and must all be there) */
Gguf *gguf_create(const char *path, char err[GGUF_ERR]);
/* one file alone: a first shard without its siblings (none opened, none required) - its metadata whole, its own
   tensors only */
Gguf *gguf_header(const char *path, char err[GGUF_ERR]);
/* the Gguf and everything it owns; NULL is nothing to do */
void gguf_destroy(Gguf *g);

/* by exact name; NULL when absent. Pointers into the Gguf, valid until gguf_destroy. */
const GgufTensor *gguf_tensor(const Gguf *g, const char *name);
const GgufKv *gguf_kv(const Gguf *g, const char *key);
/* the bytes `values` values take in `type` (whole blocks); 0 for a type not known here or a count that is not whole
   blocks */
uint64_t gguf_bytes(uint32_t type, uint64_t values);
/* an integer of any of the eight integer types: a scalar's value (i ignored), or an array's item i (i < n). false for
   another type, an index past the array, or an unsigned value past int64's range. */
bool gguf_int(const GgufKv *kv, size_t i, int64_t *out);

#ifdef __cplusplus
}
#endif

#endif
