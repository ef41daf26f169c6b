/* TEST INFRASTRUCTURE ONLY -- never linked into, imported by or executed from the product.
 *
 * Builds the reference's own CPU nn kernels into a callable shared object without a Lua VM.
 * The generic kernel files are pulled in from where they lie in the reference tree exactly
 * the way the reference's mcw_nn/init.c:1-9 instantiates them (torch_/nn_ name macros +
 * THGenerateFloatTypes.h), so every `static int nn_Float<Op>_<method>(lua_State*)` below is
 * the reference's unmodified code, including its batch loops, resizes and argument checks:
 *   mcw_nn/generic/SpatialConvolutionMM.c   (stride-1 im2col+addmm conv, the oracle for conv)
 *   mcw_nn/generic/SpatialConvolution.c     (stride-capable conv2Dmm route, used for dW/dH > 1)
 *   mcw_nn/generic/SpatialMaxPooling.c      (window max + 1-based window-local argmax)
 *   mcw_nn/generic/Threshold.c              (ReLU = Threshold(0,0))
 *   mcw_nn/generic/LogSoftMax.c             (classifier tail)
 *   mcw_nn/generic/SoftMax.c, SpatialAveragePooling.c
 * The Lua side is faked by ref_shim/lua.h: this file supplies the handful of luaT_* / luaL_*
 * functions those kernels call, reading from a flat record instead of a Lua stack. */
#include "TH.h"
#include "luaT.h"
#include <string.h>

#define torch_(NAME) TH_CONCAT_3(torch_, Real, NAME)
#define torch_Tensor TH_CONCAT_STRING_3(torch., Real, Tensor)
#define nn_(NAME) TH_CONCAT_3(nn_, Real, NAME)

#include "generic/SpatialConvolutionMM.c"
#include "THGenerateFloatTypes.h"

#include "generic/SpatialConvolution.c"
#include "THGenerateFloatTypes.h"

#include "generic/SpatialMaxPooling.c"
#include "THGenerateFloatTypes.h"

#include "generic/Threshold.c"
#include "THGenerateFloatTypes.h"

#include "generic/LogSoftMax.c"
#include "THGenerateFloatTypes.h"

#include "generic/SoftMax.c"
#include "THGenerateFloatTypes.h"

#include "generic/SpatialAveragePooling.c"
#include "THGenerateFloatTypes.h"

/* ---- fake Lua surface ------------------------------------------------------------- */

static void oref_raise(lua_State *L, const char *msg)
{
  snprintf(L->errmsg, sizeof(L->errmsg), "%s", msg ? msg : "error");
  longjmp(L->on_error, 1);
}

void lua_settop(lua_State *L, int idx) { (void)L; (void)idx; }

int luaL_argerror(lua_State *L, int numarg, const char *extramsg)
{
  char buf[400];
  snprintf(buf, sizeof(buf), "bad argument #%d (%s)", numarg, extramsg ? extramsg : "");
  oref_raise(L, buf);
  return 0;
}

lua_Number luaL_optnumber(lua_State *L, int narg, lua_Number def)
{
  if (narg >= 0 && narg < OREF_MAX_ARGS && L->arg_has_num[narg]) return L->arg_num[narg];
  return def;
}

static int oref_find(lua_State *L, const char *field)
{
  int i;
  for (i = 0; i < L->nfields; i++)
    if (strcmp(L->fields[i].name, field) == 0) return i;
  {
    char buf[200];
    snprintf(buf, sizeof(buf), "bad argument #1 (field %s does not exist)", field);
    oref_raise(L, buf);
  }
  return -1;
}

void *luaT_checkudata(lua_State *L, int ud, const char *tname)
{
  (void)tname;
  if (ud < 0 || ud >= OREF_MAX_ARGS || !L->arg_ud[ud]) luaL_argerror(L, ud, "userdata expected");
  return L->arg_ud[ud];
}
void *luaT_getfieldcheckudata(lua_State *L, int ud, const char *field, const char *tname)
{
  (void)ud; (void)tname;
  return L->fields[oref_find(L, field)].ud;
}
double luaT_getfieldchecknumber(lua_State *L, int ud, const char *field)
{
  (void)ud;
  return L->fields[oref_find(L, field)].num;
}
int luaT_getfieldcheckint(lua_State *L, int ud, const char *field)
{
  (void)ud;
  return (int)L->fields[oref_find(L, field)].num;
}
int luaT_pushmetatable(lua_State *L, const char *tname) { (void)L; (void)tname; return 1; }
void luaT_registeratname(lua_State *L, const struct luaL_Reg *methods, const char *name)
{ (void)L; (void)methods; (void)name; }

/* ---- exported driver -------------------------------------------------------------- */

lua_State *oref_state_new(void) { return (lua_State *)calloc(1, sizeof(lua_State)); }
void oref_state_free(lua_State *L) { free(L); }
const char *oref_errmsg(lua_State *L) { return L->errmsg; }

static int oref_slot(lua_State *L, const char *name)
{
  int i;
  for (i = 0; i < L->nfields; i++)
    if (strcmp(L->fields[i].name, name) == 0) return i;
  if (L->nfields >= OREF_MAX_FIELDS) return -1;
  L->fields[L->nfields].name = name; /* caller keeps the string alive */
  return L->nfields++;
}
int oref_set_num(lua_State *L, const char *name, double v)
{ int i = oref_slot(L, name); if (i < 0) return -1; L->fields[i].num = v; return 0; }
int oref_set_ud(lua_State *L, const char *name, void *p)
{ int i = oref_slot(L, name); if (i < 0) return -1; L->fields[i].ud = p; return 0; }
void oref_set_arg_ud(lua_State *L, int idx, void *p) { L->arg_ud[idx] = p; }
void oref_set_arg_num(lua_State *L, int idx, double v) { L->arg_num[idx] = v; L->arg_has_num[idx] = 1; }
void oref_clear_arg_num(lua_State *L, int idx) { L->arg_has_num[idx] = 0; }

static void oref_th_error(const char *msg, void *data) { oref_raise((lua_State *)data, msg); }
static void oref_th_argerror(int argNumber, const char *msg, void *data)
{ luaL_argerror((lua_State *)data, argNumber, msg); }

static const struct { const char *name; lua_CFunction fn; } oref_table[] = {
  {"SpatialConvolutionMM_updateOutput", nn_FloatSpatialConvolutionMM_updateOutput},
  {"SpatialConvolutionMM_updateGradInput", nn_FloatSpatialConvolutionMM_updateGradInput},
  {"SpatialConvolutionMM_accGradParameters", nn_FloatSpatialConvolutionMM_accGradParameters},
  {"SpatialConvolution_updateOutput", nn_FloatSpatialConvolution_updateOutput},
  {"SpatialConvolution_updateGradInput", nn_FloatSpatialConvolution_updateGradInput},
  {"SpatialConvolution_accGradParameters", nn_FloatSpatialConvolution_accGradParameters},
  {"SpatialMaxPooling_updateOutput", nn_FloatSpatialMaxPooling_updateOutput},
  {"SpatialMaxPooling_updateGradInput", nn_FloatSpatialMaxPooling_updateGradInput},
  {"Threshold_updateOutput", nn_FloatThreshold_updateOutput},
  {"Threshold_updateGradInput", nn_FloatThreshold_updateGradInput},
  {"LogSoftMax_updateOutput", nn_FloatLogSoftMax_updateOutput},
  {"LogSoftMax_updateGradInput", nn_FloatLogSoftMax_updateGradInput},
  {"SoftMax_updateOutput", nn_FloatSoftMax_updateOutput},
  {"SoftMax_updateGradInput", nn_FloatSoftMax_updateGradInput},
  {"SpatialAveragePooling_updateOutput", nn_FloatSpatialAveragePooling_updateOutput},
  {"SpatialAveragePooling_updateGradInput", nn_FloatSpatialAveragePooling_updateGradInput},
  {NULL, NULL}
};

/* Runs one of the reference's Lua-facing Float kernels on the record `L`.
 * Returns 0 on success, -1 when the reference raised (message via oref_errmsg),
 * -2 for an unknown name. */
int oref_call(lua_State *L, const char *name)
{
  int i;
  for (i = 0; oref_table[i].name; i++) {
    if (strcmp(oref_table[i].name, name) == 0) {
      int rc = 0;
      THSetErrorHandler(oref_th_error, L);
      THSetArgErrorHandler(oref_th_argerror, L);
      if (setjmp(L->on_error) == 0) oref_table[i].fn(L);
      else rc = -1;
      THSetErrorHandler(NULL, NULL);
      THSetArgErrorHandler(NULL, NULL);
      return rc;
    }
  }
  return -2;
}
