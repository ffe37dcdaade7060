-- xmake build of the three libraries, for maintainers who build the reference with xmake and want these
-- drop-ins from the same tool:   xmake f --cuda_arch=sm_100a && xmake && xmake install
-- Same target names, option name and install layout ($INFINI_ROOT/{lib,include}, default ~/.infini) as the
-- reference's xmake.lua:93-98,493-663.  There is one backend only (NVIDIA, sm_100a): no --nv-gpu / --cpu
-- switches, no other vendors.
--
-- NOT EXERCISED: xmake is not installed where this library is developed and tested; the build that is run
-- there (and by __graft_entry__.build) is infinicore_b200/build.py, which issues the same nvcc commands:
-- one -c per file listed below with the flags below, one -shared link per library.  Keep the two lists in step.

set_project("infinicore_b200")
set_languages("cxx17")
add_rules("mode.release")
set_policy("build.cuda.devlink", false) -- no relocatable device code: every .cu file is self-contained

option("cuda_arch")
    set_default("sm_100a")
    set_showmenu(true)
    set_description("CUDA GPU architecture; only sm_100a is supported (tcgen05, TMA and mbarrier code paths)")
    set_values("sm_100a")
    set_category("option")
option_end()

local csrc = "infinicore_b200/csrc"

-- what every CUDA translation unit is compiled with (infinicore_b200/build.py: COMMON + ARCH_FLAGS)
local function cuda_target_settings()
    add_includedirs("include", csrc)
    add_cugencodes("arch=compute_100a,code=sm_100a")
    add_cuflags("-O3", "-lineinfo", "--expt-relaxed-constexpr", {force = true})
    add_cuflags("-Xcompiler=-fPIC", "-Xcompiler=-fvisibility=hidden", "-Xcompiler=-Wall", {force = true})
    add_culdflags("-Xcompiler=-fPIC", {force = true})
    add_links("cudart")
    set_installdir(os.getenv("INFINI_ROOT") or (os.getenv("HOME") .. "/.infini"))
end

target("infinirt")
    set_kind("shared")
    cuda_target_settings()
    add_files(csrc .. "/runtime/infinirt.cu")
    add_syslinks("dl")
    add_installfiles("include/infinirt.h", {prefixdir = "include"})
    add_installfiles("include/infinicore.h", {prefixdir = "include"})
target_end()

target("infiniop")
    set_kind("shared")
    add_deps("infinirt")
    cuda_target_settings()
    add_files(csrc .. "/handle.cu", csrc .. "/kernel_status.cu")
    add_files(csrc .. "/paged_caching/paged_caching.cu")
    add_files(csrc .. "/paged_attention/operator.cu", csrc .. "/paged_attention/decode_generic.cu",
              csrc .. "/paged_attention/decode_stream.cu", csrc .. "/paged_attention/static_workspace.cu",
              csrc .. "/paged_attention/decode_step.cu")
    add_files(csrc .. "/rope/rope.cu", csrc .. "/kv_caching/kv_caching.cu")
    add_files(csrc .. "/paged_attention_prefill/operator.cu", csrc .. "/paged_attention_prefill/prefill_generic.cu",
              csrc .. "/paged_attention_prefill/prefill_tiles.cu", csrc .. "/paged_attention_prefill/prefill_umma.cu")
    add_rpathdirs("$ORIGIN")
    add_installfiles("include/infiniop/(**/*.h)", {prefixdir = "include/infiniop"})
    add_installfiles("include/infiniop/*.h", {prefixdir = "include/infiniop"})
    add_installfiles("include/infiniop.h", {prefixdir = "include"})
    add_installfiles("include/infinicore_b200/*.hpp", {prefixdir = "include/infinicore_b200"})
target_end()

target("infiniccl")
    set_kind("shared")
    add_deps("infinirt")
    cuda_target_settings()
    add_files(csrc .. "/ccl/infiniccl.cu")
    add_links("nccl")
    add_rpathdirs("$ORIGIN")
    add_installfiles("include/infiniccl.h", {prefixdir = "include"})
target_end()

-- as in the reference (xmake.lua:665-669): one name for "all three"
target("infinicore_c_api")
    set_kind("phony")
    add_deps("infiniop", "infinirt", "infiniccl")
target_end()
