/* TEST INFRASTRUCTURE ONLY: the fake Lua behind lua.h / lauxlib.h / luaT.h of this directory, and the driver the
 * tests call through ctypes (fl_*). */
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "luaT.h"

int luaopen_libgpunn(lua_State *L);
int luaopen_libgputorch(lua_State *L);

static void fl_raise(lua_State *L, const char *msg) {
  snprintf(L->errmsg, sizeof(L->errmsg), "%s", msg ? msg : "error");
  if (!L->armed) { fprintf(stderr, "fake lua: error outside a protected call: %s\n", L->errmsg); abort(); }
  longjmp(L->on_error, 1);
}

/* ---- lua.h ---- */
void lua_settop(lua_State *L, int idx) {
  if (idx < 0) {               /* lua_pop(L, n): drop pushed markers */
    int n = -idx - 1;
    while (n-- > 0 && L->nstack > 0) L->nstack--;
  }                            /* lua_settop(L, 1) in the copy methods: "return self"; nothing to model */
}
void lua_pushnumber(lua_State *L, lua_Number n) {
  if (L->nresults < 4) L->results[L->nresults++] = n;
}
void lua_newtable(lua_State *L) {
  if (L->nstack < FL_MAX_STACK) L->stack[L->nstack++] = "<table>";
}

/* ---- lauxlib.h ---- */
int luaL_error(lua_State *L, const char *fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  fl_raise(L, buf);
  return 0;
}
int luaL_argerror(lua_State *L, int numarg, const char *extramsg) {
  return luaL_error(L, "bad argument #%d (%s)", numarg, extramsg ? extramsg : "");
}
int luaL_typerror(lua_State *L, int narg, const char *tname) {
  return luaL_error(L, "bad argument #%d (%s expected)", narg, tname);
}
lua_Number luaL_optnumber(lua_State *L, int narg, lua_Number def) {
  if (narg >= 0 && narg < FL_MAX_ARGS && L->args[narg].kind == 1) return L->args[narg].num;
  return def;
}
lua_Number luaL_checknumber(lua_State *L, int narg) {
  if (narg < 0 || narg >= FL_MAX_ARGS || L->args[narg].kind != 1) luaL_typerror(L, narg, "number");
  return L->args[narg].num;
}
static void fl_register(lua_State *L, const char *owner, const char *sub, const luaL_Reg *l) {
  for (; l->name; l++) {
    if (L->nfuncs >= FL_MAX_FUNCS) fl_raise(L, "fake lua: function registry full");
    snprintf(L->funcs[L->nfuncs].owner, sizeof(L->funcs[L->nfuncs].owner), "%s%s%s", owner, sub ? "." : "", sub ? sub : "");
    L->funcs[L->nfuncs].name = l->name;
    L->funcs[L->nfuncs].fn = l->func;
    L->nfuncs++;
  }
}
void luaL_register(lua_State *L, const char *libname, const luaL_Reg *l) {
  (void)libname;
  if (L->nstack == 0) fl_raise(L, "fake lua: luaL_register with nothing on the stack");
  fl_register(L, L->stack[L->nstack - 1], NULL, l);
}

/* ---- luaT.h ---- */
void *luaT_toudata(lua_State *L, int ud, const char *tname) {
  if (ud < 0 || ud >= FL_MAX_ARGS || L->args[ud].kind != 2) return NULL;
  return strcmp(L->args[ud].tname, tname) == 0 ? L->args[ud].ud : NULL;
}
void *luaT_checkudata(lua_State *L, int ud, const char *tname) {
  void *p = luaT_toudata(L, ud, tname);
  if (!p) luaL_typerror(L, ud, tname);
  return p;
}
static int fl_find(lua_State *L, const char *field) {
  for (int i = 0; i < L->nfields; i++)
    if (strcmp(L->fields[i].name, field) == 0) return i;
  luaL_error(L, "bad argument #1 (field %s does not exist)", field);
  return -1;
}
void *luaT_getfieldcheckudata(lua_State *L, int ud, const char *field, const char *tname) {
  (void)ud;
  const int i = fl_find(L, field);
  if (L->fields[i].kind != 2 || strcmp(L->fields[i].tname, tname) != 0)
    luaL_error(L, "bad argument #1 (field %s is not a %s)", field, tname);
  return L->fields[i].ud;
}
double luaT_getfieldchecknumber(lua_State *L, int ud, const char *field) {
  (void)ud;
  const int i = fl_find(L, field);
  if (L->fields[i].kind != 1) luaL_error(L, "bad argument #1 (field %s is not a number)", field);
  return L->fields[i].num;
}
int luaT_getfieldcheckint(lua_State *L, int ud, const char *field) { return (int)luaT_getfieldchecknumber(L, ud, field); }
int luaT_getfieldcheckboolean(lua_State *L, int ud, const char *field) {
  (void)ud;
  const int i = fl_find(L, field);
  if (L->fields[i].kind != 3) luaL_error(L, "bad argument #1 (field %s is not a boolean)", field);
  return L->fields[i].num != 0;
}
int luaT_pushmetatable(lua_State *L, const char *tname) {
  if (L->nstack < FL_MAX_STACK) L->stack[L->nstack++] = tname;
  return 1;
}
void luaT_registeratname(lua_State *L, const struct luaL_Reg *methods, const char *name) {
  if (L->nstack == 0) fl_raise(L, "fake lua: luaT_registeratname with nothing on the stack");
  fl_register(L, L->stack[L->nstack - 1], name, methods);
}

/* ---- driver (called from the tests) ---- */
lua_State *fl_new(void) { return (lua_State *)calloc(1, sizeof(lua_State)); }
void fl_free(lua_State *L) { free(L); }
const char *fl_errmsg(lua_State *L) { return L->errmsg; }
void fl_clear_call(lua_State *L) {
  memset(L->args, 0, sizeof(L->args));
  L->nfields = 0;
  L->nresults = 0;
}
void fl_arg_ud(lua_State *L, int idx, void *p, const char *tname) { L->args[idx].kind = 2; L->args[idx].ud = p; L->args[idx].tname = tname; }
void fl_arg_num(lua_State *L, int idx, double v) { L->args[idx].kind = 1; L->args[idx].num = v; }
static int fl_slot(lua_State *L, const char *name) {
  for (int i = 0; i < L->nfields; i++)
    if (strcmp(L->fields[i].name, name) == 0) return i;
  if (L->nfields >= FL_MAX_FIELDS) return -1;
  L->fields[L->nfields].name = name;   /* the caller keeps the string alive */
  return L->nfields++;
}
int fl_field_num(lua_State *L, const char *name, double v) { int i = fl_slot(L, name); if (i < 0) return -1; L->fields[i].kind = 1; L->fields[i].num = v; return 0; }
int fl_field_bool(lua_State *L, const char *name, int v) { int i = fl_slot(L, name); if (i < 0) return -1; L->fields[i].kind = 3; L->fields[i].num = v; return 0; }
int fl_field_ud(lua_State *L, const char *name, void *p, const char *tname) {
  int i = fl_slot(L, name); if (i < 0) return -1;
  L->fields[i].kind = 2; L->fields[i].ud = p; L->fields[i].tname = tname; return 0;
}
/* Runs luaopen_libgpunn (which = 0) or luaopen_libgputorch (1); returns its result count, -1 on a Lua error. */
int fl_open(lua_State *L, int which) {
  int rc;
  L->armed = 1;
  if (setjmp(L->on_error) == 0) rc = which == 0 ? luaopen_libgpunn(L) : luaopen_libgputorch(L);
  else rc = -1;
  L->armed = 0;
  return rc;
}
int fl_registered(lua_State *L) { return L->nfuncs; }
const char *fl_registered_owner(lua_State *L, int i) { return L->funcs[i].owner; }
const char *fl_registered_name(lua_State *L, int i) { return L->funcs[i].name; }
/* Calls the function registered as owner / name with the arguments and fields set before.  Returns the number of
 * Lua results, -1 when it raised (message via fl_errmsg), -2 when nothing is registered under that name. */
int fl_call(lua_State *L, const char *owner, const char *name) {
  for (int i = 0; i < L->nfuncs; i++) {
    if (strcmp(L->funcs[i].owner, owner) == 0 && strcmp(L->funcs[i].name, name) == 0) {
      int rc;
      L->nresults = 0;
      L->armed = 1;
      if (setjmp(L->on_error) == 0) rc = L->funcs[i].fn(L);
      else rc = -1;
      L->armed = 0;
      return rc;
    }
  }
  return -2;
}
double fl_result(lua_State *L, int i) { return L->results[i]; }
