/* TEST INFRASTRUCTURE ONLY (checker for tests / smoke / the bench's CPU baseline leg).
 *
 * Minimal stand-in for the Lua 5.1 C API, just wide enough for the reference's CPU nn
 * kernels (mcw_nn/generic/*.c) to compile and run UNMODIFIED without a Lua VM.  The
 * reference functions only ever (a) fetch typed userdata from stack slots 2/3, (b) fetch
 * named fields of the module table in slot 1, (c) read an optional number in slot 4 and
 * (d) raise argument errors.  A `lua_State` here is therefore a flat record: positional
 * userdata pointers, optional numbers, and a small name -> {number | pointer} table. */
#ifndef ORACLE_REF_SHIM_LUA_H
#define ORACLE_REF_SHIM_LUA_H
#include <setjmp.h>
#include <stddef.h>

typedef double lua_Number;

#define OREF_MAX_FIELDS 48
#define OREF_MAX_ARGS 8

typedef struct lua_State {
  struct { const char *name; double num; void *ud; } fields[OREF_MAX_FIELDS];
  int nfields;
  void *arg_ud[OREF_MAX_ARGS];
  double arg_num[OREF_MAX_ARGS];
  int arg_has_num[OREF_MAX_ARGS];
  jmp_buf on_error;
  char errmsg[512];
} lua_State;

typedef int (*lua_CFunction)(lua_State *L);

void lua_settop(lua_State *L, int idx);
#define lua_pop(L, n) lua_settop(L, -(n)-1)
#endif
