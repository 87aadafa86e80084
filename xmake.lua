-- xmake build of libllaisys (the reference's build tool; see llaisys_b200/build.py for the g++/nvcc build that
-- is exercised where xmake is not installed). Same option name as the reference: `xmake f --nv-gpu=y`.
add_rules("mode.debug", "mode.release")
set_encodings("utf-8")
set_languages("cxx17")
add_includedirs("include", "llaisys_b200/csrc")

option("nv-gpu")
    set_default(false)
    set_showmenu(true)
    set_description("Build the NVIDIA (sm_100a) backend")
option_end()

if has_config("nv-gpu") then
    add_defines("ENABLE_NVIDIA_API")
    includes("xmake/nvidia.lua")
end

target("llaisys")
    set_kind("shared")
    set_warnings("all", "error")
    add_cxflags("-fPIC", "-fvisibility=hidden", "-fopenmp")
    add_ldflags("-fopenmp")
    add_files("llaisys_b200/csrc/**.cpp", "llaisys_b200/csrc/**.cc")
    if has_config("nv-gpu") then
        add_deps("llaisys-nvidia")
    end
    set_installdir(".")
    after_build(function (target)
        -- the ctypes loader looks next to llaisys_b200/libllaisys/__init__.py
        os.cp(target:targetfile(), "llaisys_b200/libllaisys/libllaisys.so")
    end)
target_end()
