-- CUDA part of libllaisys: device runtime table and the sm_100a kernels (append/gather, split-KV decode with
-- cp.async and with TMA, generic attention, LSE merge). sm_100a only: the explicit gencode emits no generic
-- compute_100 PTX, which would reject the tcgen05 / TMA instructions.
target("llaisys-nvidia")
    set_kind("static")
    set_languages("cxx17")
    add_rules("cuda")
    set_policy("build.cuda.devlink", true)
    add_includedirs("../include", "../llaisys_b200/csrc")
    add_defines("ENABLE_NVIDIA_API")
    add_files("../llaisys_b200/csrc/**.cu")
    add_cuflags("-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler=-fPIC,-fvisibility=hidden", {force = true})
    add_cugencodes("arch=compute_100a,code=sm_100a")
    add_culdflags("-gencode arch=compute_100a,code=sm_100a", {force = true})
    add_links("cudart_static", "dl", "rt", "pthread")
    on_install(function (target) end)
target_end()
