"""TEST INFRASTRUCTURE: builds oracle/_ref/liboracle_refnet.so -- the reference's whole CPU library (cfg parser, .weights
loader, fuse_conv_batchnorm, calculate_binary_weights, every layer's CPU forward, yolo / region decoding, NMS), compiled
unmodified from the mounted darknet tree, plus refnet_glue.cpp.  The reference's build system is not run; the OpenCV
stand-in under ref_stub/ supplies the names its sources mention.  Translation units that are all windows, image files,
charts or the command line are left out; whatever the others still reference from them is bound to an aborting stub.

    python oracle/build_refnet.py            # needs the reference tree (DARKNET_REFERENCE_DIR or the default mount)
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from oracle.binding import reference_dir  # noqa: E402

OUT = os.path.join(HERE, "_ref", "net")
LIB = os.path.join(HERE, "_ref", "liboracle_refnet.so")
LEFT_OUT = {"Chart", "image_opencv", "darknet_image", "nightmare", "yolo_v2_class", "darknet", "amd_rocm"}
FLAGS = ["-std=c++17", "-O2", "-mavx2", "-mfma", "-mpopcnt", "-fopenmp", "-DDARKNET_OPENMP", "-fPIC", "-w"]


def build(force: bool = False) -> str:
    ref = reference_dir()
    src_dir = os.path.join(ref, "src-lib")
    if not os.path.isdir(src_dir):
        raise FileNotFoundError("reference tree not mounted")
    gen = os.path.join(HERE, "_ref", "gen")
    if not os.path.exists(os.path.join(gen, "darknet_version.h")):
        subprocess.check_call(["make", "-C", HERE, "ref", f"REF={ref}"], stdout=subprocess.DEVNULL)
    os.makedirs(OUT, exist_ok=True)
    inc = ["-I", os.path.join(HERE, "ref_stub"), "-I", gen, "-I", src_dir, "-I", os.path.join(ref, "src-other")]
    jobs = [(s, os.path.join(OUT, os.path.basename(s)[:-4] + ".o")) for s in sorted(glob.glob(os.path.join(src_dir, "*.cpp")))
            if os.path.basename(s)[:-4] not in LEFT_OUT]
    jobs.append((os.path.join(HERE, "refnet_glue.cpp"), os.path.join(OUT, "refnet_glue.o")))
    stub = os.path.join(HERE, "ref_stub", "opencv2", "opencv.hpp")

    def compile_one(job):
        src, obj = job
        if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(src), os.path.getmtime(stub)):
            return None
        r = subprocess.run(["g++"] + FLAGS + inc + ["-c", src, "-o", obj], capture_output=True, text=True)
        return None if r.returncode == 0 else f"{src}:\n{r.stderr[-2000:]}"

    with cf.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        errors = [e for e in ex.map(compile_one, jobs) if e]
    if errors:
        raise RuntimeError("reference sources failed to compile:\n" + "\n".join(errors))
    objs = [o for _, o in jobs]
    link = ["g++", "-shared", "-fopenmp", "-o", LIB, "-Wl,--no-demangle", "-Wl,--no-undefined"] + objs
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        missing = sorted(set(re.findall(r"undefined reference to `([A-Za-z0-9_.$]+)'", r.stderr)))
        if not missing:
            raise RuntimeError(r.stderr[-3000:])
        link += [f"-Wl,--defsym,{sym}=refnet_unreachable" for sym in missing]
        subprocess.check_call(link)
        print(f"{len(missing)} reference symbols from left-out translation units bound to refnet_unreachable")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
