/* TEST INFRASTRUCTURE ONLY: a stand-in for the Lua 5.1 C API, just wide enough to compile and drive the library's
 * Lua glue (the C files under mcw_cppamp_torch_b200/lua) on machines that have no Lua.  A lua_State is a flat record:
 *   - positional arguments (slot 1 is the module table, whose fields live in `fields`),
 *   - a small stack of "what was pushed" markers (a new table, a metatable by type name) that luaL_register and
 *     luaT_registeratname write into,
 *   - the registry of every C function registered so far, by owner ("torch.GPUTensor", "torch.GPUTensor.nn",
 *     "<table>") and name, which the driver (fake_lua.c: fl_call) looks functions up in,
 *   - numbers pushed as results, and the error message + jump buffer luaL_error leaves through. */
#ifndef TEST_LUA_SHIM_LUA_H
#define TEST_LUA_SHIM_LUA_H
#include <setjmp.h>
#include <stddef.h>

typedef double lua_Number;
struct lua_State;
typedef struct lua_State lua_State;
typedef int (*lua_CFunction)(lua_State *L);

#define FL_MAX_ARGS 8
#define FL_MAX_FIELDS 48
#define FL_MAX_FUNCS 128
#define FL_MAX_STACK 8

struct lua_State {
  struct { int kind; double num; void *ud; const char *tname; } args[FL_MAX_ARGS];        /* kind: 0 nil, 1 number, 2 userdata */
  struct { const char *name; int kind; double num; void *ud; const char *tname; } fields[FL_MAX_FIELDS]; /* 3: boolean */
  int nfields;
  const char *stack[FL_MAX_STACK];   /* "<table>" or a type name */
  int nstack;
  struct { char owner[64]; const char *name; lua_CFunction fn; } funcs[FL_MAX_FUNCS];
  int nfuncs;
  double results[4];
  int nresults;
  jmp_buf on_error;
  int armed;
  char errmsg[1024];
};

void lua_settop(lua_State *L, int idx);
#define lua_pop(L, n) lua_settop(L, -(n)-1)
void lua_pushnumber(lua_State *L, lua_Number n);
void lua_newtable(lua_State *L);
#endif
