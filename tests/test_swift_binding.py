"""The Swift-side files (swiftlm_b200/swift/, written without a Swift toolchain) against the C header they
bind: the header copy inside the SwiftPM C target is the header, the module map names it, and every
dflash_* call in the Swift sources passes exactly as many arguments as the header's prototype declares."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SWIFT = os.path.join(ROOT, "swiftlm_b200", "swift")
HEADER = os.path.join(ROOT, "include", "dflash_cuda.h")


def _strip_c_comments(text):
    return re.sub(r"/\*.*?\*/", "", text, flags=re.S)


def header_prototypes():
    text = _strip_c_comments(open(HEADER).read())
    protos = {}
    for m in re.finditer(r"\b(dflash_\w+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S):
        name, args = m.group(1), m.group(2).strip()
        protos[name] = 0 if args in ("", "void") else len(args.split(","))
    return protos


def _split_top_level(args):
    parts, depth, cur = [], 0, ""
    for ch in args:
        if ch in "([{":
            depth += 1
        elif ch in ")]}":
            depth -= 1
        if ch == "," and depth == 0:
            parts.append(cur)
            cur = ""
        else:
            cur += ch
    if cur.strip():
        parts.append(cur)
    return parts


def swift_calls(path):
    text = open(path).read()
    text = re.sub(r"//[^\n]*", "", text)
    out = []
    for m in re.finditer(r"\b(dflash_\w+)\s*\(", text):
        i, depth = m.end(), 1
        while depth and i < len(text):
            depth += text[i] in "([{"
            depth -= text[i] in ")]}"
            i += 1
        out.append((m.group(1), len(_split_top_level(text[m.end():i - 1]))))
    return out


def test_header_copy_in_the_swiftpm_target_is_the_header():
    copy = os.path.join(SWIFT, "Sources", "CDFlashCUDA", "include", "dflash_cuda.h")
    assert open(copy).read() == open(HEADER).read(), "re-copy include/dflash_cuda.h into the SwiftPM C target"
    mm = open(os.path.join(SWIFT, "Sources", "CDFlashCUDA", "include", "module.modulemap")).read()
    assert 'header "dflash_cuda.h"' in mm and 'link "dflash_cuda"' in mm and "module CDFlashCUDA" in mm


def test_every_swift_call_matches_the_prototype():
    protos = header_prototypes()
    assert protos["dflash_verify_sdpa"] == 22 and protos["dflash_tape_replay"] == 17 and protos["dflash_gated_delta_tape"] == 21
    seen = set()
    for dirpath, _, files in os.walk(SWIFT):
        for f in files:
            if not f.endswith(".swift"):
                continue
            for name, nargs in swift_calls(os.path.join(dirpath, f)):
                assert name in protos, f"{f}: {name} is not declared in dflash_cuda.h"
                assert nargs == protos[name], f"{f}: {name} called with {nargs} arguments, the header declares {protos[name]}"
                seen.add(name)
    # the three kernel entry points of the path are bound
    assert {"dflash_tape_replay", "dflash_gated_delta_tape", "dflash_verify_sdpa", "dflash_verify_sdpa_workspace_bytes"} <= seen


def test_manifest_patch_names_the_c_target_and_its_users():
    patch = open(os.path.join(SWIFT, "Package.swift.patch")).read()
    assert 'name: "CDFlashCUDA"' in patch and patch.count('+                "CDFlashCUDA",') == 2
    kpatch = open(os.path.join(SWIFT, "Sources", "DFlash", "DFlashKernels.swift.patch")).read()
    for fn in ("DFlashCUDA.tapeReplay(", "DFlashCUDA.gatedDeltaWithTape(", "DFlashCUDA.batchedSDPA2Pass("):
        assert fn in kpatch
    assert "precondition" not in open(os.path.join(SWIFT, "Sources", "DFlash", "DFlashCUDA.swift")).read()
