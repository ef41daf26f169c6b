/* TEST INFRASTRUCTURE ONLY: stand-in for torch's luaT.h (mcw_torch7_core/lib/luaT/luaT.h); see lua.h beside it. */
#ifndef TEST_LUA_SHIM_LUAT_H
#define TEST_LUA_SHIM_LUAT_H
#include "lauxlib.h"

void *luaT_checkudata(lua_State *L, int ud, const char *tname);
void *luaT_toudata(lua_State *L, int ud, const char *tname);
void *luaT_getfieldcheckudata(lua_State *L, int ud, const char *field, const char *tname);
double luaT_getfieldchecknumber(lua_State *L, int ud, const char *field);
int luaT_getfieldcheckint(lua_State *L, int ud, const char *field);
int luaT_getfieldcheckboolean(lua_State *L, int ud, const char *field);
int luaT_pushmetatable(lua_State *L, const char *tname);
void luaT_registeratname(lua_State *L, const struct luaL_Reg *methods, const char *name);
#endif
