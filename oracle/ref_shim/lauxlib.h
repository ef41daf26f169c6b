/* TEST INFRASTRUCTURE ONLY. Stand-in for Lua's lauxlib.h; see lua.h beside it. */
#ifndef ORACLE_REF_SHIM_LAUXLIB_H
#define ORACLE_REF_SHIM_LAUXLIB_H
#include "lua.h"

typedef struct luaL_Reg { const char *name; lua_CFunction func; } luaL_Reg;

int luaL_argerror(lua_State *L, int numarg, const char *extramsg);
lua_Number luaL_optnumber(lua_State *L, int narg, lua_Number def);
#define luaL_argcheck(L, cond, numarg, extramsg) \
  ((void)((cond) || luaL_argerror(L, (numarg), (extramsg))))
#endif
