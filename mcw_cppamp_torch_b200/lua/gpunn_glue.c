/* Lua-facing glue of the gpunn operators: libgpunn.so / open_libgpunn for Torch7.
 *
 * Each `static int gpunn_<Op>_<method>(lua_State *L)` keeps the protocol of its namesake in the reference
 * (gputorch/lib/THC/gpunn-impl/<Op>.cpp): stack slot 1 is the module table, 2 the input, 3 gradOutput (or the
 * criterion's target), 4 the optional scale; hyper-parameters and state tensors are fetched BY FIELD NAME from
 * slot 1; results are written in place into the module's tensors; the return value is the number of Lua results
 * the reference returns (1, or 0 for accGradParameters).  The bodies only forward to the plain-C cores
 * THGPUNN_<Op>_<method> of libTHC.so.  A core that fails has recorded a message; it is raised with luaL_error,
 * which leaves by longjmp, so no function here holds anything that needs unwinding.
 *
 * The functions are registered exactly as the reference registers them: under the `nn` sub-table of the
 * "torch.GPUTensor" metatable (luaT_pushmetatable + luaT_registeratname, e.g. SpatialConvolutionMM.cpp:431-443),
 * so that `input.nn.SpatialConvolutionMM_updateOutput(self, input)` of the unmodified mcw_nn Lua modules
 * dispatches here when `input` is a torch.GPUTensor.
 *
 * Builds against Lua 5.1 / LuaJIT + luaT headers:
 *   cc -shared -fPIC -I<lua> -I<luaT> -I include gpunn_glue.c -L. -lTHC -lluaT -o libgpunn.so            */
#include <stdio.h>

#include <lua.h>
#include <lauxlib.h>
#include <luaT.h>

#include "THC.h"

#define GPU "torch.GPUTensor"

static THGPUTensor *arg_tensor(lua_State *L, int slot) { return (THGPUTensor *)luaT_checkudata(L, slot, GPU); }
static THGPUTensor *field_tensor(lua_State *L, const char *name) {
  return (THGPUTensor *)luaT_getfieldcheckudata(L, 1, name, GPU);
}
/* turns the status of a core into the Lua result count, or raises its message */
static int finish(lua_State *L, int status, int nresults) {
  if (status != 0) {
    const char *msg = THGPUGetLastError();
    char copy[1024];
    snprintf(copy, sizeof(copy), "%s", msg ? msg : "gpunn: operation failed");
    THGPUClearError();
    return luaL_error(L, "%s", copy);
  }
  return nresults;
}

/* ---- SpatialConvolutionMM (gpunn-impl/SpatialConvolutionMM.cpp:110-128, :227-244, :313-331) ---- */
static int gpunn_SpatialConvolutionMM_updateOutput(lua_State *L) {
  THGPUTensor *input = arg_tensor(L, 2);
  int dW = luaT_getfieldcheckint(L, 1, "dW");
  int dH = luaT_getfieldcheckint(L, 1, "dH");
  int kW = luaT_getfieldcheckint(L, 1, "kW");
  int kH = luaT_getfieldcheckint(L, 1, "kH");
  int nInputPlane = luaT_getfieldcheckint(L, 1, "nInputPlane");
  int nOutputPlane = luaT_getfieldcheckint(L, 1, "nOutputPlane");
  int padding = luaT_getfieldcheckint(L, 1, "padding");
  THGPUTensor *weight = field_tensor(L, "weight");
  THGPUTensor *bias = field_tensor(L, "bias");
  THGPUTensor *finput = field_tensor(L, "finput");
  THGPUTensor *fgradInput = field_tensor(L, "fgradInput");
  THGPUTensor *output = field_tensor(L, "output");
  luaL_argcheck(L, input->nDimension == 3 || input->nDimension == 4, 2, "3D or 4D (batch mode) tensor is expected");
  luaL_argcheck(L, input->size[input->nDimension - 3] == nInputPlane, 2, "input channels and nInputPlane dont match");
  luaL_argcheck(L, weight->nDimension == 2 && weight->size[0] == nOutputPlane, 1, "weight and nOutputPlane dont match");
  return finish(L, THGPUNN_SpatialConvolutionMM_updateOutput(input, output, weight, bias, finput, fgradInput, kW, kH, dW, dH,
                                                             padding), 1);
}
static int gpunn_SpatialConvolutionMM_updateGradInput(lua_State *L) {
  THGPUTensor *input = arg_tensor(L, 2);
  THGPUTensor *gradOutput = arg_tensor(L, 3);
  int dW = luaT_getfieldcheckint(L, 1, "dW");
  int dH = luaT_getfieldcheckint(L, 1, "dH");
  int kW = luaT_getfieldcheckint(L, 1, "kW");
  int kH = luaT_getfieldcheckint(L, 1, "kH");
  int nInputPlane = luaT_getfieldcheckint(L, 1, "nInputPlane");
  int padding = luaT_getfieldcheckint(L, 1, "padding");
  THGPUTensor *weight = field_tensor(L, "weight");
  THGPUTensor *finput = field_tensor(L, "finput");
  THGPUTensor *fgradInput = field_tensor(L, "fgradInput");
  THGPUTensor *gradInput = field_tensor(L, "gradInput");
  luaL_argcheck(L, input->nDimension == 3 || input->nDimension == 4, 2, "3D or 4D (batch mode) tensor is expected");
  luaL_argcheck(L, input->size[input->nDimension - 3] == nInputPlane, 2, "input channels and nInputPlane dont match");
  return finish(L, THGPUNN_SpatialConvolutionMM_updateGradInput(input, gradOutput, gradInput, weight, finput, fgradInput, kW, kH,
                                                                dW, dH, padding), 1);
}
static int gpunn_SpatialConvolutionMM_accGradParameters(lua_State *L) {
  THGPUTensor *input = arg_tensor(L, 2);
  THGPUTensor *gradOutput = arg_tensor(L, 3);
  int dW = luaT_getfieldcheckint(L, 1, "dW");
  int dH = luaT_getfieldcheckint(L, 1, "dH");
  int kW = luaT_getfieldcheckint(L, 1, "kW");
  int kH = luaT_getfieldcheckint(L, 1, "kH");
  int nInputPlane = luaT_getfieldcheckint(L, 1, "nInputPlane");
  int padding = luaT_getfieldcheckint(L, 1, "padding");
  float scale = (float)luaL_optnumber(L, 4, 1);
  THGPUTensor *gradWeight = field_tensor(L, "gradWeight");
  THGPUTensor *gradBias = field_tensor(L, "gradBias");
  THGPUTensor *finput = field_tensor(L, "finput");
  THGPUTensor *fgradInput = field_tensor(L, "fgradInput");
  luaL_argcheck(L, input->nDimension == 3 || input->nDimension == 4, 2, "3D or 4D (batch mode) tensor is expected");
  luaL_argcheck(L, input->size[input->nDimension - 3] == nInputPlane, 2, "input channels and nInputPlane dont match");
  return finish(L, THGPUNN_SpatialConvolutionMM_accGradParameters(input, gradOutput, gradWeight, gradBias, finput, fgradInput, kW,
                                                                  kH, dW, dH, padding, scale), 0);
}
static const struct luaL_Reg gpunn_SpatialConvolutionMM__[] = {
  {"SpatialConvolutionMM_updateOutput", gpunn_SpatialConvolutionMM_updateOutput},
  {"SpatialConvolutionMM_updateGradInput", gpunn_SpatialConvolutionMM_updateGradInput},
  {"SpatialConvolutionMM_accGradParameters", gpunn_SpatialConvolutionMM_accGradParameters},
  {NULL, NULL}
};

/* ---- SpatialMaxPooling (gpunn-impl/SpatialMaxPooling.cpp:205-214, :283-298; overlapping windows are accepted) ---- */
static int gpunn_SpatialMaxPooling_updateOutput(lua_State *L) {
  THGPUTensor *input = arg_tensor(L, 2);
  int kW = luaT_getfieldcheckint(L, 1, "kW");
  int kH = luaT_getfieldcheckint(L, 1, "kH");
  int dW = luaT_getfieldcheckint(L, 1, "dW");
  int dH = luaT_getfieldcheckint(L, 1, "dH");
  THGPUTensor *output = field_tensor(L, "output");
  THGPUTensor *indices = field_tensor(L, "indices");
  return finish(L, THGPUNN_SpatialMaxPooling_updateOutput(input, output, indices, kW, kH, dW, dH), 1);
}
static int gpunn_SpatialMaxPooling_updateGradInput(lua_State *L) {
  THGPUTensor *input = arg_tensor(L, 2);
  THGPUTensor *gradOutput = arg_tensor(L, 3);
  int kW = luaT_getfieldcheckint(L, 1, "kW");
  int kH = luaT_getfieldcheckint(L, 1, "kH");
  int dW = luaT_getfieldcheckint(L, 1, "dW");
  int dH = luaT_getfieldcheckint(L, 1, "dH");
  THGPUTensor *gradInput = field_tensor(L, "gradInput");
  THGPUTensor *indices = field_tensor(L, "indices");
  return finish(L, THGPUNN_SpatialMaxPooling_updateGradInput(input, gradOutput, gradInput, indices, kW, kH, dW, dH), 1);
}
static const struct luaL_Reg gpunn_SpatialMaxPooling__[] = {
  {"SpatialMaxPooling_updateOutput", gpunn_SpatialMaxPooling_updateOutput},
  {"SpatialMaxPooling_updateGradInput", gpunn_SpatialMaxPooling_updateGradInput},
  {NULL, NULL}
};

/* ---- Threshold (gpunn-impl/Threshold.cpp:16-22, :53-61) ---- */
static int gpunn_Threshold_updateOutput(lua_State *L) {
  THGPUTensor *input = arg_tensor(L, 2);
  THGPUTensor *output = field_tensor(L, "output");
  double val = luaT_getfieldchecknumber(L, 1, "val");
  double threshold = luaT_getfieldchecknumber(L, 1, "threshold");
  return finish(L, THGPUNN_Threshold_updateOutput(input, output, threshold, val), 1);
}
static int gpunn_Threshold_updateGradInput(lua_State *L) {
  THGPUTensor *input = arg_tensor(L, 2);
  THGPUTensor *gradOutput = arg_tensor(L, 3);
  THGPUTensor *gradInput = field_tensor(L, "gradInput");
  double threshold = luaT_getfieldchecknumber(L, 1, "threshold");
  return finish(L, THGPUNN_Threshold_updateGradInput(input, gradOutput, gradInput, threshold), 1);
}
static const struct luaL_Reg gpunn_Threshold__[] = {
  {"Threshold_updateOutput", gpunn_Threshold_updateOutput},
  {"Threshold_updateGradInput", gpunn_Threshold_updateGradInput},
  {NULL, NULL}
};

/* ---- LogSoftMax (gpunn-impl/LogSoftMax.cpp:116-119, :146-150) and SoftMax (gpunn-impl/SoftMax.cpp) ---- */
static int gpunn_LogSoftMax_updateOutput(lua_State *L) {
  THGPUTensor *input = arg_tensor(L, 2);
  THGPUTensor *output = field_tensor(L, "output");
  return finish(L, THGPUNN_LogSoftMax_updateOutput(input, output), 1);
}
static int gpunn_LogSoftMax_updateGradInput(lua_State *L) {
  THGPUTensor *input = arg_tensor(L, 2);
  THGPUTensor *gradOutput = arg_tensor(L, 3);
  THGPUTensor *output = field_tensor(L, "output");
  THGPUTensor *gradInput = field_tensor(L, "gradInput");
  return finish(L, THGPUNN_LogSoftMax_updateGradInput(input, gradOutput, gradInput, output), 1);
}
static int gpunn_SoftMax_updateOutput(lua_State *L) {
  THGPUTensor *input = arg_tensor(L, 2);
  THGPUTensor *output = field_tensor(L, "output");
  return finish(L, THGPUNN_SoftMax_updateOutput(input, output), 1);
}
static int gpunn_SoftMax_updateGradInput(lua_State *L) {
  THGPUTensor *input = arg_tensor(L, 2);
  THGPUTensor *gradOutput = arg_tensor(L, 3);
  THGPUTensor *output = field_tensor(L, "output");
  THGPUTensor *gradInput = field_tensor(L, "gradInput");
  return finish(L, THGPUNN_SoftMax_updateGradInput(input, gradOutput, gradInput, output), 1);
}
static const struct luaL_Reg gpunn_SoftMaxes__[] = {
  {"LogSoftMax_updateOutput", gpunn_LogSoftMax_updateOutput},
  {"LogSoftMax_updateGradInput", gpunn_LogSoftMax_updateGradInput},
  {"SoftMax_updateOutput", gpunn_SoftMax_updateOutput},
  {"SoftMax_updateGradInput", gpunn_SoftMax_updateGradInput},
  {NULL, NULL}
};

/* ---- SpatialAveragePooling (gpunn-impl/SpatialAveragePooling.cpp:66-75, :184-197) ---- */
static int gpunn_SpatialAveragePooling_updateOutput(lua_State *L) {
  THGPUTensor *input = arg_tensor(L, 2);
  int kW = luaT_getfieldcheckint(L, 1, "kW");
  int kH = luaT_getfieldcheckint(L, 1, "kH");
  int dW = luaT_getfieldcheckint(L, 1, "dW");
  int dH = luaT_getfieldcheckint(L, 1, "dH");
  THGPUTensor *output = field_tensor(L, "output");
  return finish(L, THGPUNN_SpatialAveragePooling_updateOutput(input, output, kW, kH, dW, dH), 1);
}
static int gpunn_SpatialAveragePooling_updateGradInput(lua_State *L) {
  THGPUTensor *input = arg_tensor(L, 2);
  THGPUTensor *gradOutput = arg_tensor(L, 3);
  int kW = luaT_getfieldcheckint(L, 1, "kW");
  int kH = luaT_getfieldcheckint(L, 1, "kH");
  int dW = luaT_getfieldcheckint(L, 1, "dW");
  int dH = luaT_getfieldcheckint(L, 1, "dH");
  THGPUTensor *gradInput = field_tensor(L, "gradInput");
  return finish(L, THGPUNN_SpatialAveragePooling_updateGradInput(input, gradOutput, gradInput, kW, kH, dW, dH), 1);
}
static const struct luaL_Reg gpunn_SpatialAveragePooling__[] = {
  {"SpatialAveragePooling_updateOutput", gpunn_SpatialAveragePooling_updateOutput},
  {"SpatialAveragePooling_updateGradInput", gpunn_SpatialAveragePooling_updateGradInput},
  {NULL, NULL}
};

/* ---- ClassNLLCriterion (gpunn-impl/ClassNLLCriterion.cpp:96-134, :137-185): slot 3 is the target, a GPU tensor of
 * 1-based class ids; the loss lands in the module's `outputTensor`, which the Lua side reads back ---- */
static int gpunn_ClassNLLCriterion_updateOutput(lua_State *L) {
  THGPUTensor *input = arg_tensor(L, 2);
  THGPUTensor *target = arg_tensor(L, 3);
  THGPUTensor *output = field_tensor(L, "outputTensor");
  int sizeAverage = luaT_getfieldcheckboolean(L, 1, "sizeAverage");
  return finish(L, THGPUNN_ClassNLLCriterion_updateOutput(input, target, output, sizeAverage), 1);
}
static int gpunn_ClassNLLCriterion_updateGradInput(lua_State *L) {
  THGPUTensor *input = arg_tensor(L, 2);
  THGPUTensor *target = arg_tensor(L, 3);
  THGPUTensor *gradInput = field_tensor(L, "gradInput");
  int sizeAverage = luaT_getfieldcheckboolean(L, 1, "sizeAverage");
  return finish(L, THGPUNN_ClassNLLCriterion_updateGradInput(input, target, gradInput, sizeAverage), 1);
}
static const struct luaL_Reg gpunn_ClassNLLCriterion__[] = {
  {"ClassNLLCriterion_updateOutput", gpunn_ClassNLLCriterion_updateOutput},
  {"ClassNLLCriterion_updateGradInput", gpunn_ClassNLLCriterion_updateGradInput},
  {NULL, NULL}
};

static void register_nn(lua_State *L, const struct luaL_Reg *methods) {
  luaT_pushmetatable(L, GPU);
  luaT_registeratname(L, methods, "nn");
  lua_pop(L, 1);
}

/* gputorch/lib/THC/gpunn-impl/init.cpp:34-65 (the operators of this library's path) */
int open_libgpunn(lua_State *L) {
  register_nn(L, gpunn_SoftMaxes__);
  register_nn(L, gpunn_SpatialConvolutionMM__);
  register_nn(L, gpunn_SpatialMaxPooling__);
  register_nn(L, gpunn_Threshold__);
  register_nn(L, gpunn_SpatialAveragePooling__);
  register_nn(L, gpunn_ClassNLLCriterion__);
  return 1;
}

/* gpunn/init.cpp:5-11 */
int luaopen_libgpunn(lua_State *L) { return open_libgpunn(L); }
