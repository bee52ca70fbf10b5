# Package configuration of the B200 build of bitsqz_llm for CMake consumers.
#
# The reference installs a package that downstream projects use as
#     find_package(bitsqz_llm CONFIG REQUIRED)
#     target_link_libraries(app PRIVATE bitsqz_llm::bitsqz_llm)
# (CMakeLists.txt:74-124 and README.md:287-299 of the reference).  This file gives the same target name for the
# shared library built in this tree by `python bitsqueeze-llm_b200/build.py` (lib/libbitsqz_llm.so, sm_100a), so such a
# project switches over by pointing bitsqz_llm_DIR (or CMAKE_PREFIX_PATH) at this directory; nothing is copied or
# installed.  The target carries the public headers (include/bitsqz_llm.hpp with the reference's interface,
# include/bitsqz_llm_c.h with the C ABI).
get_filename_component(_bsq_pkg_dir "${CMAKE_CURRENT_LIST_DIR}/.." ABSOLUTE)
get_filename_component(_bsq_root "${_bsq_pkg_dir}/.." ABSOLUTE)
set(_bsq_lib "${_bsq_pkg_dir}/lib/libbitsqz_llm.so")
if(NOT EXISTS "${_bsq_lib}")
    set(bitsqz_llm_FOUND FALSE)
    set(bitsqz_llm_NOT_FOUND_MESSAGE "${_bsq_lib} has not been built: run python bitsqueeze-llm_b200/build.py")
    return()
endif()
if(NOT TARGET bitsqz_llm::bitsqz_llm)
    add_library(bitsqz_llm::bitsqz_llm SHARED IMPORTED)
    set_target_properties(bitsqz_llm::bitsqz_llm PROPERTIES
        IMPORTED_LOCATION "${_bsq_lib}"
        IMPORTED_SONAME "libbitsqz_llm.so"
        INTERFACE_INCLUDE_DIRECTORIES "${_bsq_root}/include"
        INTERFACE_COMPILE_FEATURES cxx_std_17)
endif()
set(bitsqz_llm_VERSION 0.2.0)
set(bitsqz_llm_INCLUDE_DIRS "${_bsq_root}/include")
set(bitsqz_llm_LIBRARIES bitsqz_llm::bitsqz_llm)
unset(_bsq_lib)
unset(_bsq_pkg_dir)
unset(_bsq_root)
