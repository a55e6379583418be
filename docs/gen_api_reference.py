"""Regenerates docs/api_reference.md from the public headers: python docs/gen_api_reference.py (from the repository root)."""
import re, pathlib
inc = pathlib.Path('csrc/include/hccl')
out = ["# API reference (generated from the public headers)", "",
       "Every exported function of `csrc/include/hccl/*.h`, by header. All return `HcclResult` unless the signature says",
       "otherwise; `hcclStream_t` is a `cudaStream_t`. The comments in the headers give semantics and ownership; `api_overview.md`",
       "gives the conventions.", ""]
order = ["hccl.h", "hccl_comm.h", "hccl_types.h", "hccl_ext.h", "hccl_graph_mode.h", "hccl_mc2.h", "hccl_moe.h", "hccl_moe_noalloc.h", "hccl_fused_ops.h",
         "hccl_tuner_plugin.h", "hccl_algo_plugin.h"]
total = 0
for name in order:
    text = (inc / name).read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    protos = re.findall(r"^(?!static|typedef|#)([A-Za-z_][\w \*]*?\b(Hccl\w+|GetHcclAlgoPlugin))\s*\(([^;{}]*?)\)\s*;", text, flags=re.M | re.S)
    if not protos:
        continue
    out += [f"## `{name}`", "", "| Function | Parameters |", "|---|---|"]
    for full, fn, args in protos:
        ret = full[:full.rfind(fn)].strip()
        args = " ".join(args.split())
        sig = f"`{fn}`" + ("" if ret == "HcclResult" else f" → `{ret}`")
        out.append(f"| {sig} | `{args or 'void'}` |")
        total += 1
    out.append("")
out.insert(5, f"{total} functions.")
pathlib.Path('docs/api_reference.md').write_text("\n".join(out) + "\n")
print(total)
