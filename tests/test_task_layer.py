"""The C++ task layer (src/cupynumeric/sort/sort.cu: the GPU variant of the SORT task over the C
ABI) must keep compiling against the header: a syntax check with stand-in Legate declarations."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_task_body_compiles_against_the_header():
    cmd = ["g++", "-std=c++17", "-fsyntax-only", "-Wall", "-x", "c++", "-DB2S_SYNTAX_CHECK", "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(ROOT, "src", "third_party_stubs"), os.path.join(ROOT, "src", "cupynumeric", "sort", "sort.cu")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_task_body_calls_only_declared_entry_points():
    import re

    body = open(os.path.join(ROOT, "src", "cupynumeric", "sort", "sort.cu")).read()
    header = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "b200sort.h")).read(), flags=re.S)
    declared = set(re.findall(r"\b(b2s_[a-z0-9_]+)\s*\(", header))
    used = set(re.findall(r"\b(b2s_[a-z0-9_]+)\s*\(", re.sub(r"//.*", "", body))) - {"b2s_code", "b2s_check"}
    assert used and used <= declared, used - declared
