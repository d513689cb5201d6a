# Build entry of the cuda_sm100 backend: one complete, independent source graph.
# Selected through the catalog (backends/targets.json -> build_entry) the same way the
# reference selects cmake/backends/sm90.cmake from cmake/GdnBackend.cmake:56-71.
if(NOT GDN_QSA_RESOLVED_TARGET STREQUAL "cuda_sm100")
  message(FATAL_ERROR "SM100 source graph rejects ${GDN_QSA_RESOLVED_TARGET}")
endif()
find_package(Python3 REQUIRED COMPONENTS Interpreter)
set(GDN_SM100_COMPILER "" CACHE FILEPATH "Explicit sm_100a-capable nvcc (CUDA >= 12.8)")
set(_sm100_args --out ${CMAKE_CURRENT_BINARY_DIR}/sm100)
if(GDN_SM100_COMPILER)
  list(APPEND _sm100_args --compiler ${GDN_SM100_COMPILER})
endif()
get_filename_component(_sm100_package "${CMAKE_CURRENT_LIST_DIR}/../.." ABSOLUTE)
get_filename_component(_sm100_root "${_sm100_package}/.." ABSOLUTE)
add_custom_target(gdn_wy_sm100 ALL
  COMMAND ${CMAKE_COMMAND} -E env "PYTHONPATH=${_sm100_root}"
    ${Python3_EXECUTABLE} -m actlizela_b200.build_sm100 ${_sm100_args}
  WORKING_DIRECTORY ${_sm100_root} USES_TERMINAL)
