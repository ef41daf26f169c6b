/* Lua-facing glue of the gputorch package: luaopen_libgputorch, the device functions and the cross-type `copy`
 * methods (gputorch/init.cpp:10-94, gputorch/Tensor.cpp:37-231, gputorch/Storage.cpp:39-120).
 *
 * What is here: the `gputorch` table (synchronize, getDevice, setDevice, getDeviceCount -- empty stubs in the
 * reference, real here; device numbers are 1-based on the Lua side), and the `copy` method of every tensor and
 * storage type, which probes the type of its argument with luaT_toudata and forwards to THGPUTensor_copy<Type> /
 * TH<Type>Tensor_copyGPU exactly as the reference dispatches.  `x:gpu()`, `x:float()`, `x:double()` of
 * gputorch/Tensor.lua are `new + resize + copy` on top of these.
 *
 * What is not here: the object methods of torch.GPUStorage / torch.GPUTensor that the reference generates from
 * torch's generic/Storage.c, generic/Tensor.c and the cwrap math tables (gputorch/TensorMath.cpp); those files
 * are instantiated for the GPU type by the same `#define real float / #define Real GPU` recipe against this
 * library's THC.h, which exports every THGPUTensor_* / THGPUStorage_* symbol they call.
 *
 * Builds against Lua 5.1 / LuaJIT + luaT headers:
 *   cc -shared -fPIC -I<lua> -I<luaT> -I include gputorch_glue.c -L. -lTHC -lluaT -o libgputorch.so     */
#include <stdio.h>

#include <lua.h>
#include <lauxlib.h>
#include <luaT.h>

#include "THC.h"

static void raise_pending(lua_State *L) {
  const char *msg = THGPUGetLastError();
  if (msg) {
    char copy[1024];
    snprintf(copy, sizeof(copy), "%s", msg);
    THGPUClearError();
    luaL_error(L, "%s", copy);
  }
}

static int gputorch_synchronize(lua_State *L) {
  THGPUSynchronize();
  raise_pending(L);
  return 0;
}
static int gputorch_getDevice(lua_State *L) {
  int d = THGPUGetDevice();
  raise_pending(L);
  lua_pushnumber(L, d + 1);
  return 1;
}
static int gputorch_getDeviceCount(lua_State *L) {
  lua_pushnumber(L, THGPUGetDeviceCount());
  return 1;
}
static int gputorch_setDevice(lua_State *L) {
  int d = (int)luaL_checknumber(L, 1);
  luaL_argcheck(L, d >= 1 && d <= THGPUGetDeviceCount(), 1, "device number out of range");
  THGPUSetDevice(d - 1);
  raise_pending(L);
  return 0;
}
static const struct luaL_Reg gputorch_stuff__[] = {
  {"synchronize", gputorch_synchronize},
  {"getDevice", gputorch_getDevice},
  {"getDeviceCount", gputorch_getDeviceCount},
  {"setDevice", gputorch_setDevice},
  {NULL, NULL}
};

/* x:copy(y) for x a torch.GPUTensor: y may be a tensor of any type (gputorch/Tensor.cpp:37-65) */
static int gputorch_GPUTensor_copy(lua_State *L) {
  THGPUTensor *self = (THGPUTensor *)luaT_checkudata(L, 1, "torch.GPUTensor");
  void *src;
  if ((src = luaT_toudata(L, 2, "torch.GPUTensor"))) THGPUTensor_copy(self, (THGPUTensor *)src);
  else if ((src = luaT_toudata(L, 2, "torch.ByteTensor"))) THGPUTensor_copyByte(self, (THByteTensor *)src);
  else if ((src = luaT_toudata(L, 2, "torch.CharTensor"))) THGPUTensor_copyChar(self, (THCharTensor *)src);
  else if ((src = luaT_toudata(L, 2, "torch.ShortTensor"))) THGPUTensor_copyShort(self, (THShortTensor *)src);
  else if ((src = luaT_toudata(L, 2, "torch.IntTensor"))) THGPUTensor_copyInt(self, (THIntTensor *)src);
  else if ((src = luaT_toudata(L, 2, "torch.LongTensor"))) THGPUTensor_copyLong(self, (THLongTensor *)src);
  else if ((src = luaT_toudata(L, 2, "torch.FloatTensor"))) THGPUTensor_copyFloat(self, (THFloatTensor *)src);
  else if ((src = luaT_toudata(L, 2, "torch.DoubleTensor"))) THGPUTensor_copyDouble(self, (THDoubleTensor *)src);
  else luaL_typerror(L, 2, "torch.*Tensor");
  raise_pending(L);
  lua_settop(L, 1);
  return 1;
}
/* x:copy(y) for x a host tensor of type <Type> and y a torch.GPUTensor (gputorch/Tensor.cpp:67-105); any other
 * argument type is left to the method this one replaced, which the caller finds under `copyHost` */
#define GPU_IMPLEMENT_TENSOR_COPY(TYPEC)                                                             \
  static int gputorch_##TYPEC##Tensor_copy(lua_State *L) {                                           \
    TH##TYPEC##Tensor *self = (TH##TYPEC##Tensor *)luaT_checkudata(L, 1, "torch." #TYPEC "Tensor");  \
    void *src = luaT_toudata(L, 2, "torch.GPUTensor");                                               \
    if (!src) luaL_typerror(L, 2, "torch.GPUTensor");                                                \
    TH##TYPEC##Tensor_copyGPU(self, (THGPUTensor *)src);                                             \
    raise_pending(L);                                                                                \
    lua_settop(L, 1);                                                                                \
    return 1;                                                                                        \
  }
GPU_IMPLEMENT_TENSOR_COPY(Byte)
GPU_IMPLEMENT_TENSOR_COPY(Char)
GPU_IMPLEMENT_TENSOR_COPY(Short)
GPU_IMPLEMENT_TENSOR_COPY(Int)
GPU_IMPLEMENT_TENSOR_COPY(Long)
GPU_IMPLEMENT_TENSOR_COPY(Float)
GPU_IMPLEMENT_TENSOR_COPY(Double)

static const struct luaL_Reg gputorch_GPUTensor_copy__[] = {{"copy", gputorch_GPUTensor_copy}, {NULL, NULL}};
#define GPU_COPY_TABLE(TYPEC) \
  static const struct luaL_Reg gputorch_##TYPEC##Tensor_copy__[] = {{"copyGPU", gputorch_##TYPEC##Tensor_copy}, {NULL, NULL}};
GPU_COPY_TABLE(Byte)
GPU_COPY_TABLE(Char)
GPU_COPY_TABLE(Short)
GPU_COPY_TABLE(Int)
GPU_COPY_TABLE(Long)
GPU_COPY_TABLE(Float)
GPU_COPY_TABLE(Double)

static void set_methods(lua_State *L, const char *tname, const struct luaL_Reg *methods) {
  luaT_pushmetatable(L, tname);
  luaL_register(L, NULL, methods);
  lua_pop(L, 1);
}

int luaopen_libgputorch(lua_State *L) {
  THGPUInit();
  raise_pending(L);
  lua_newtable(L);
  luaL_register(L, NULL, gputorch_stuff__);
  set_methods(L, "torch.GPUTensor", gputorch_GPUTensor_copy__);
  set_methods(L, "torch.ByteTensor", gputorch_ByteTensor_copy__);
  set_methods(L, "torch.CharTensor", gputorch_CharTensor_copy__);
  set_methods(L, "torch.ShortTensor", gputorch_ShortTensor_copy__);
  set_methods(L, "torch.IntTensor", gputorch_IntTensor_copy__);
  set_methods(L, "torch.LongTensor", gputorch_LongTensor_copy__);
  set_methods(L, "torch.FloatTensor", gputorch_FloatTensor_copy__);
  set_methods(L, "torch.DoubleTensor", gputorch_DoubleTensor_copy__);
  return 1;
}
