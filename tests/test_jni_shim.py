"""The JNI shim compiles against a stand-in <jni.h> and keeps the JNI rules: lengths are read before arrays are
pinned, null column arrays are refused (tests/cpp/test_jni_shim.cpp runs the registration entry points against a
fake JVM; registration is host-side work, so no GPU is needed)."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "systemds_b200")


def test_jni_shim_against_fake_jvm():
    from systemds_b200 import build
    build.build()
    exe = os.path.join(ROOT, "tests", "cpp", "test_jni_shim.bin")
    cmd = ["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "tests", "cpp", "jni_stub"),
           os.path.join(ROOT, "tests", "cpp", "test_jni_shim.cpp"), os.path.join(LIBDIR, "csrc", "cla_jni.cpp"),
           "-o", exe, f"-L{LIBDIR}", "-lsystemds_cla", f"-Wl,-rpath,{LIBDIR}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    r = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "JNI SHIM OK" in r.stdout, r.stdout + r.stderr
