/* GGUF headers as data (include/osmos_b200/gguf.h): the reference's src/model/gguf.c:49-190 rebuilt around one bounded
 * reader.
 *
 * A file is read front to back through `In`: a FILE, the file's size and the position. Nothing is taken from the file
 * without `room()` having compared it with what is left - a count is checked against the least bytes its entries could
 * take before anything is allocated for it, a length against the bytes left before it is read. A failure anywhere
 * records "file: offset: what" once and unwinds through gguf_destroy, which frees a half-built Gguf as well as a whole
 * one (every pointer starts NULL, every count says how many entries are filled).
 */
#define _GNU_SOURCE
#define _FILE_OFFSET_BITS 64
#include "osmos_b200/gguf.h"

#include <errno.h>
#include <inttypes.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "osmos_b200/qtype.h"

#define GGUF_MAGIC 0x46554747u /* "GGUF" */
#define TYPE_MXFP8 43u
#define TYPE_F8_E4M3 0x12Bu /* a type-43 tensor that holds one E4M3 byte a value and no scales */

/* ---- sizes by type: the kernels' table, and what only a file holds ------------------------------------------------ */
typedef struct
{
  uint32_t id, values, bytes;
} SizeRow;
#define ROW(name, id, values, bytes, paths) {id, values, bytes},
static const SizeRow kSizes[] = {OSMOS_QTYPE_TABLE(ROW){26, 1, 4} /* I32 */, {27, 1, 8} /* I64 */, {TYPE_F8_E4M3, 1, 1}};
#undef ROW

uint64_t gguf_bytes(uint32_t type, uint64_t values)
{
  for (size_t i = 0; i < sizeof kSizes / sizeof kSizes[0]; i++)
    if (kSizes[i].id == type)
    {
      uint64_t bytes;
      if (!values || values % kSizes[i].values || __builtin_mul_overflow(values / kSizes[i].values, (uint64_t)kSizes[i].bytes, &bytes))
        return 0;
      return bytes;
    }
  return 0;
}

/* ---- the bounded reader ----------------------------------------------------------------------------------------------- */
typedef struct
{
  FILE *f;
  const char *path;
  uint64_t size, pos;
  char *err; /* GGUF_ERR bytes; the first failure wins */
  bool failed;
} In;

static bool fail(In *in, const char *fmt, ...)
{
  if (!in->failed)
  {
    in->failed = true;
    int n = snprintf(in->err, GGUF_ERR, "%s: offset %" PRIu64 ": ", in->path, in->pos);
    if (n < 0 || n >= GGUF_ERR)
      n = GGUF_ERR - 1;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(in->err + n, (size_t)(GGUF_ERR - n), fmt, ap);
    va_end(ap);
  }
  return false;
}

static bool room(In *in, uint64_t n, const char *what)
{
  if (in->failed)
    return false;
  if (n > in->size - in->pos)
    return fail(in, "%s needs %" PRIu64 " bytes, the file has %" PRIu64 " left", what, n, in->size - in->pos);
  return true;
}

static bool take(In *in, void *dst, uint64_t n, const char *what)
{
  if (!room(in, n, what))
    return false;
  if (n && fread(dst, 1, (size_t)n, in->f) != n)
    return fail(in, "%s: read error", what);
  in->pos += n;
  return true;
}

static bool take_u32(In *in, uint32_t *v, const char *what) { return take(in, v, 4, what); }
static bool take_u64(In *in, uint64_t *v, const char *what) { return take(in, v, 8, what); }

/* a length-prefixed string as a NUL-terminated copy */
static char *take_string(In *in, const char *what)
{
  uint64_t len;
  if (!take_u64(in, &len, what) || !room(in, len, what))
    return NULL;
  char *s = malloc((size_t)len + 1);
  if (!s)
  {
    fail(in, "%s: out of memory", what);
    return NULL;
  }
  if (!take(in, s, len, what))
  {
    free(s);
    return NULL;
  }
  s[len] = 0;
  return s;
}

static uint32_t scalar_width(uint32_t type)
{
  switch (type)
  {
  case GGUF_UINT8:
  case GGUF_INT8:
  case GGUF_BOOL:
    return 1;
  case GGUF_UINT16:
  case GGUF_INT16:
    return 2;
  case GGUF_UINT32:
  case GGUF_INT32:
  case GGUF_FLOAT32:
    return 4;
  case GGUF_UINT64:
  case GGUF_INT64:
  case GGUF_FLOAT64:
    return 8;
  default:
    return 0;
  }
}

/* a scalar at p, of any of the eleven scalar types, widened into the entry */
static void widen(GgufKv *kv, uint32_t type, const void *p)
{
  switch (type)
  {
  case GGUF_UINT8:
  case GGUF_BOOL:
    kv->v.u = *(const uint8_t *)p;
    break;
  case GGUF_INT8:
    kv->v.i = *(const int8_t *)p;
    break;
  case GGUF_UINT16:
  {
    uint16_t v;
    memcpy(&v, p, 2);
    kv->v.u = v;
    break;
  }
  case GGUF_INT16:
  {
    int16_t v;
    memcpy(&v, p, 2);
    kv->v.i = v;
    break;
  }
  case GGUF_UINT32:
  {
    uint32_t v;
    memcpy(&v, p, 4);
    kv->v.u = v;
    break;
  }
  case GGUF_INT32:
  {
    int32_t v;
    memcpy(&v, p, 4);
    kv->v.i = v;
    break;
  }
  case GGUF_FLOAT32:
  {
    float v;
    memcpy(&v, p, 4);
    kv->v.f = v;
    break;
  }
  case GGUF_UINT64:
    memcpy(&kv->v.u, p, 8);
    break;
  case GGUF_INT64:
    memcpy(&kv->v.i, p, 8);
    break;
  case GGUF_FLOAT64:
    memcpy(&kv->v.f, p, 8);
    break;
  default:
    break;
  }
}

static void kv_release(GgufKv *kv)
{
  free(kv->key);
  if (kv->type == GGUF_STRING)
    free(kv->v.s);
  if (kv->type == GGUF_ARRAY)
  {
    if (kv->item == GGUF_STRING && kv->v.items)
      for (uint64_t i = 0; i < kv->n; i++)
        free(((char **)kv->v.items)[i]);
    free(kv->v.items);
  }
  memset(kv, 0, sizeof *kv);
}

/* one metadata entry into *kv (zeroed by the caller); on failure what it holds is still releasable */
static bool take_kv(In *in, GgufKv *kv)
{
  uint32_t type;
  if (!(kv->key = take_string(in, "a metadata key")) || !take_u32(in, &type, "a metadata value's type"))
    return false;
  kv->type = (GgufValueType)type;
  if (scalar_width(type))
  {
    uint8_t raw[8] = {0};
    if (!take(in, raw, scalar_width(type), kv->key))
      return false;
    widen(kv, type, raw);
    return true;
  }
  if (type == GGUF_STRING)
    return (kv->v.s = take_string(in, kv->key)) != NULL;
  if (type != GGUF_ARRAY)
    return fail(in, "key %s: unknown value type %u", kv->key, type);
  uint32_t item;
  uint64_t n;
  if (!take_u32(in, &item, kv->key) || !take_u64(in, &n, kv->key))
    return false;
  kv->item = (GgufValueType)item;
  if (scalar_width(item))
  {
    uint64_t bytes;
    if (__builtin_mul_overflow(n, (uint64_t)scalar_width(item), &bytes) || !room(in, bytes, kv->key))
      return in->failed ? false : fail(in, "key %s: an array of %" PRIu64 " items overflows", kv->key, n);
    if (bytes && !(kv->v.items = malloc((size_t)bytes)))
      return fail(in, "key %s: out of memory", kv->key);
    kv->n = n;
    return take(in, kv->v.items, bytes, kv->key);
  }
  if (item != GGUF_STRING)
    return fail(in, "key %s: an array of type %u (only scalars and strings are read)", kv->key, item);
  /* n strings take at least their 8-byte lengths */
  if (n > (in->size - in->pos) / 8)
    return fail(in, "key %s: %" PRIu64 " strings cannot fit in the bytes left", kv->key, n);
  char **items = n ? calloc((size_t)n, sizeof *items) : NULL;
  if (n && !items)
    return fail(in, "key %s: out of memory", kv->key);
  kv->v.items = items;
  for (uint64_t i = 0; i < n; i++)
  {
    if (!(items[i] = take_string(in, kv->key)))
      return false;
    kv->n = i + 1; /* (what kv_release frees) */
  }
  return true;
}

/* ---- a Gguf under construction ------------------------------------------------------------------------------------ */
const GgufKv *gguf_kv(const Gguf *g, const char *key)
{
  if (g && key)
    for (size_t i = 0; i < g->n_kv; i++)
      if (!strcmp(g->kv[i].key, key))
        return &g->kv[i];
  return NULL;
}

const GgufTensor *gguf_tensor(const Gguf *g, const char *name)
{
  if (g && name)
    for (size_t i = 0; i < g->n_tensors; i++)
      if (!strcmp(g->tensors[i].name, name))
        return &g->tensors[i];
  return NULL;
}

bool gguf_int(const GgufKv *kv, size_t i, int64_t *out)
{
  if (!kv || !out)
    return false;
  uint32_t type = kv->type;
  GgufKv one = {0};
  const GgufKv *src = kv;
  if (type == GGUF_ARRAY)
  {
    type = kv->item;
    const uint32_t w = scalar_width(type);
    if (!w || type == GGUF_STRING || i >= kv->n)
      return false;
    widen(&one, type, (const uint8_t *)kv->v.items + i * w);
    src = &one;
  }
  switch (type)
  {
  case GGUF_UINT8:
  case GGUF_UINT16:
  case GGUF_UINT32:
  case GGUF_UINT64:
    if (src->v.u > (uint64_t)INT64_MAX)
      return false;
    *out = (int64_t)src->v.u;
    return true;
  case GGUF_INT8:
  case GGUF_INT16:
  case GGUF_INT32:
  case GGUF_INT64:
    *out = src->v.i;
    return true;
  default:
    return false;
  }
}

void gguf_destroy(Gguf *g)
{
  if (!g)
    return;
  for (int i = 0; i < g->n_files; i++)
    free(g->paths[i]);
  free(g->paths);
  free(g->sizes);
  for (size_t i = 0; i < g->n_kv; i++)
    kv_release(&g->kv[i]);
  free(g->kv);
  for (size_t i = 0; i < g->n_tensors; i++)
    free(g->tensors[i].name);
  free(g->tensors);
  free(g);
}

/* One file's header into g as its shard `file`: the metadata kept when `keep_kv` (the first shard's), the tensors
   appended. *split_count: the file's split.count (0 when it has none). */
static bool read_file(Gguf *g, const char *path, int file, bool keep_kv, int64_t *split_no, int64_t *split_count, char *err)
{
  In in = {fopen(path, "rb"), path, 0, 0, err, false};
  if (!in.f)
    return fail(&in, "cannot open: %s", strerror(errno));
  bool ok = false;
  GgufKv *tmp_kv = NULL; /* a sibling shard's metadata: read (its lengths must hold), then dropped */
  uint64_t n_tmp = 0;
  if (fseeko(in.f, 0, SEEK_END) || (in.size = (uint64_t)ftello(in.f), fseeko(in.f, 0, SEEK_SET)))
  {
    fail(&in, "cannot find the file's size");
    goto done;
  }
  g->paths[file] = strdup(path);
  g->sizes[file] = in.size;
  if (!g->paths[file])
  {
    fail(&in, "out of memory");
    goto done;
  }
  g->n_files = file + 1;

  uint32_t magic, version;
  uint64_t n_tensors, n_kv;
  if (!take_u32(&in, &magic, "the magic") || !take_u32(&in, &version, "the version"))
    goto done;
  if (magic != GGUF_MAGIC)
  {
    fail(&in, "not a GGUF file (magic %08x)", magic);
    goto done;
  }
  if (version != 2 && version != 3)
  {
    fail(&in, "GGUF version %u (2 and 3 are read)", version);
    goto done;
  }
  if (!take_u64(&in, &n_tensors, "the tensor count") || !take_u64(&in, &n_kv, "the metadata count"))
    goto done;
  /* an entry takes at least a key's length and a type (12 bytes), a tensor a name's length, dims, type, offset (24) */
  if (n_kv > (in.size - in.pos) / 12 || n_tensors > (in.size - in.pos) / 24)
  {
    fail(&in, "%" PRIu64 " metadata entries and %" PRIu64 " tensors cannot fit in the file", n_kv, n_tensors);
    goto done;
  }

  GgufKv **kvs = keep_kv ? &g->kv : &tmp_kv;
  uint64_t filled = 0;
  if (n_kv && !(*kvs = calloc((size_t)n_kv, sizeof **kvs)))
  {
    fail(&in, "out of memory");
    goto done;
  }
  for (; filled < n_kv; filled++)
  {
    const bool good = take_kv(&in, &(*kvs)[filled]);
    if (keep_kv)
      g->n_kv = (size_t)filled + 1;
    else
      n_tmp = filled + 1;
    if (!good)
      goto done;
  }
  Gguf view = {0}; /* this file's metadata, for the three keys read here */
  view.kv = *kvs, view.n_kv = (size_t)n_kv;
  int64_t align = 32;
  const GgufKv *ka = gguf_kv(&view, "general.alignment");
  if (ka && (!gguf_int(ka, 0, &align) || align <= 0 || align > (1 << 20) || (align & (align - 1))))
  {
    fail(&in, "general.alignment is not a power of two up to 2^20");
    goto done;
  }
  *split_no = 0, *split_count = 0;
  const GgufKv *kc = gguf_kv(&view, "split.count"), *kn = gguf_kv(&view, "split.no");
  if (kc && (!gguf_int(kc, 0, split_count) || *split_count < 0 || *split_count > 99999))
  {
    fail(&in, "split.count is not a count of shards");
    goto done;
  }
  if (kn && !gguf_int(kn, 0, split_no))
  {
    fail(&in, "split.no is not an integer");
    goto done;
  }

  /* the tensors: appended to the model's */
  const size_t first = g->n_tensors;
  if (n_tensors)
  {
    GgufTensor *grown = realloc(g->tensors, (first + (size_t)n_tensors) * sizeof *grown);
    if (!grown)
    {
      fail(&in, "out of memory");
      goto done;
    }
    g->tensors = grown;
    memset(grown + first, 0, (size_t)n_tensors * sizeof *grown);
  }
  for (uint64_t i = 0; i < n_tensors; i++)
  {
    GgufTensor *t = &g->tensors[first + i];
    if (!(t->name = take_string(&in, "a tensor's name")))
      goto done;
    g->n_tensors = first + (size_t)i + 1;
    if (!take_u32(&in, &t->n_dims, t->name))
      goto done;
    if (t->n_dims < 1 || t->n_dims > GGUF_MAX_DIMS)
    {
      fail(&in, "tensor %s: %u dimensions", t->name, t->n_dims);
      goto done;
    }
    for (uint32_t d = 0; d < t->n_dims; d++)
      if (!take_u64(&in, &t->dims[d], t->name))
        goto done;
    if (!take_u32(&in, &t->type, t->name) || !take_u64(&in, &t->offset, t->name))
      goto done;
    t->file = file;
    for (size_t j = 0; j + 1 < g->n_tensors; j++)
      if (!strcmp(g->tensors[j].name, t->name))
      {
        fail(&in, "tensor %s: the name is there twice", t->name);
        goto done;
      }
  }
  /* the data section starts at the next multiple of the alignment; a tensor's offset counts from there */
  const uint64_t data0 = (in.pos + (uint64_t)align - 1) / (uint64_t)align * (uint64_t)align;
  for (size_t i = first; i < g->n_tensors; i++)
  {
    GgufTensor *t = &g->tensors[i];
    uint64_t values = 1;
    for (uint32_t d = 0; d < t->n_dims; d++)
      if (!t->dims[d] || __builtin_mul_overflow(values, t->dims[d], &values))
      {
        fail(&in, "tensor %s: its dimensions multiply past 64 bits (or one is 0)", t->name);
        goto done;
      }
    if (data0 > in.size || t->offset > in.size - data0)
    {
      fail(&in, "tensor %s: its data starts past the file's end", t->name);
      goto done;
    }
    const uint64_t at = data0 + t->offset;
    /* its room: up to the next tensor's start in this file, or the file's end */
    uint64_t end = in.size;
    for (size_t j = first; j < g->n_tensors; j++)
    {
      const uint64_t o = g->tensors[j].offset; /* (still relative for j > i, already absolute for j < i: compare both ways) */
      const uint64_t abs_j = j < i ? o : data0 + (o <= in.size - data0 ? o : in.size - data0);
      if (j != i && abs_j > at && abs_j < end)
        end = abs_j;
    }
    uint64_t bytes = gguf_bytes(t->type, values);
    if (t->type == TYPE_MXFP8 && (!bytes || bytes > end - at) && values <= end - at)
      t->type = TYPE_F8_E4M3, bytes = values; /* a type 43 that fits only a byte a value: upstream's F8_E4M3 */
    if (!bytes)
    {
      fail(&in, "tensor %s: type %u with %" PRIu64 " values (an unknown type, or not whole blocks)", t->name, t->type, values);
      goto done;
    }
    if (bytes > in.size - at)
    {
      fail(&in, "tensor %s: %" PRIu64 " bytes at %" PRIu64 " leave the file (%" PRIu64 " bytes)", t->name, bytes, at, in.size);
      goto done;
    }
    t->offset = at, t->bytes = bytes;
  }
  ok = true;
done:
  for (uint64_t i = 0; i < n_tmp; i++)
    kv_release(&tmp_kv[i]);
  free(tmp_kv);
  if (in.f)
    fclose(in.f);
  return ok && !in.failed;
}

/* the path of shard `no` (1-based) of `count`, given the first shard's path "<stem>-00001-of-<count as 5 digits>.gguf";
   NULL when the path does not have that form */
static char *shard_path(const char *first, int64_t no, int64_t count)
{
  char tail[32];
  snprintf(tail, sizeof tail, "-00001-of-%05" PRId64 ".gguf", count);
  const size_t n = strlen(first), m = strlen(tail);
  if (n < m || strcmp(first + n - m, tail))
    return NULL;
  char *p = malloc(n + 1);
  if (!p)
    return NULL;
  memcpy(p, first, n + 1);
  char num[8];
  snprintf(num, sizeof num, "%05" PRId64, no);
  memcpy(p + n - m + 1, num, 5);
  return p;
}

static Gguf *open_model(const char *path, bool with_siblings, char err[GGUF_ERR])
{
  char local[GGUF_ERR];
  if (!err)
    err = local;
  err[0] = 0;
  if (!path)
  {
    snprintf(err, GGUF_ERR, "no path");
    return NULL;
  }
  Gguf *g = calloc(1, sizeof *g);
  int cap = 1;
  if (g)
    g->paths = calloc((size_t)cap, sizeof *g->paths), g->sizes = calloc((size_t)cap, sizeof *g->sizes);
  if (!g || !g->paths || !g->sizes)
  {
    snprintf(err, GGUF_ERR, "%s: out of memory", path);
    gguf_destroy(g);
    return NULL;
  }
  int64_t no = 0, count = 0;
  if (!read_file(g, path, 0, true, &no, &count, err))
  {
    gguf_destroy(g);
    return NULL;
  }
  if (with_siblings && count > 1)
  {
    if (no != 0)
    {
      snprintf(err, GGUF_ERR, "%s: shard %" PRId64 " of a split model (open its first)", path, no + 1);
      gguf_destroy(g);
      return NULL;
    }
    char **paths = realloc(g->paths, (size_t)count * sizeof *paths);
    if (paths)
      g->paths = paths, memset(paths + 1, 0, (size_t)(count - 1) * sizeof *paths);
    uint64_t *sizes = paths ? realloc(g->sizes, (size_t)count * sizeof *sizes) : NULL;
    if (sizes)
      g->sizes = sizes;
    if (!paths || !sizes)
    {
      snprintf(err, GGUF_ERR, "%s: out of memory", path);
      gguf_destroy(g);
      return NULL;
    }
    for (int64_t s = 1; s < count; s++)
    {
      char *sp = shard_path(path, s + 1, count);
      int64_t sno = 0, scount = 0;
      bool ok = sp && read_file(g, sp, (int)s, false, &sno, &scount, err);
      if (!sp)
        snprintf(err, GGUF_ERR, "%s: a split model's first shard is named <stem>-00001-of-%05" PRId64 ".gguf", path, count);
      else if (ok && (sno != s || scount != count))
      {
        snprintf(err, GGUF_ERR, "%s: says it is shard %" PRId64 " of %" PRId64 ", expected %" PRId64 " of %" PRId64, sp, sno + 1,
                 scount, s + 1, count);
        ok = false;
      }
      free(sp);
      if (!ok)
      {
        gguf_destroy(g);
        return NULL;
      }
    }
  }
  return g;
}

Gguf *gguf_create(const char *path, char err[GGUF_ERR]) { return open_model(path, true, err); }
Gguf *gguf_header(const char *path, char err[GGUF_ERR]) { return open_model(path, false, err); }
