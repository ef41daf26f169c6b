/* TEST INFRASTRUCTURE ONLY: stand-in for Lua's lauxlib.h; see lua.h beside it. */
#ifndef TEST_LUA_SHIM_LAUXLIB_H
#define TEST_LUA_SHIM_LAUXLIB_H
#include "lua.h"

typedef struct luaL_Reg { const char *name; lua_CFunction func; } luaL_Reg;

int luaL_error(lua_State *L, const char *fmt, ...);
int luaL_argerror(lua_State *L, int numarg, const char *extramsg);
int luaL_typerror(lua_State *L, int narg, const char *tname);
lua_Number luaL_optnumber(lua_State *L, int narg, lua_Number def);
lua_Number luaL_checknumber(lua_State *L, int narg);
void luaL_register(lua_State *L, const char *libname, const luaL_Reg *l);
#define luaL_argcheck(L, cond, numarg, extramsg) ((void)((cond) || luaL_argerror(L, (numarg), (extramsg))))
#endif
