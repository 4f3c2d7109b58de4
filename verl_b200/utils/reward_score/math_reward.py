"""MATH-style scoring: compare the last \\boxed{...} of the solution with the ground truth after normalisation."""

import re


def last_boxed_only_string(s: str):
    idx = s.rfind("\\boxed")
    if idx < 0:
        idx = s.rfind("\\fbox")
        if idx < 0:
            return None
    depth, end = 0, None
    for i in range(idx, len(s)):
        if s[i] == "{":
            depth += 1
        elif s[i] == "}":
            depth -= 1
            if depth == 0:
                end = i
                break
    return s[idx : end + 1] if end is not None else None


def remove_boxed(s: str) -> str:
    if s.startswith("\\boxed "):
        return s[len("\\boxed "):]
    left = "\\boxed{"
    assert s.startswith(left) and s.endswith("}"), s
    return s[len(left):-1]


def _fix_fracs(s: str) -> str:
    parts = s.split("\\frac")
    out = parts[0]
    for p in parts[1:]:
        out += "\\frac"
        if p and p[0] != "{":
            if len(p) < 2:
                return s
            a, b, rest = p[0], p[1], p[2:]
            out += "{" + a + "}" + ("{" + b + "}" + rest if b != "{" else b + rest)
        else:
            out += p
    return out


def _fix_sqrt(s: str) -> str:
    return re.sub(r"\\sqrt(\w)", r"\\sqrt{\1}", s)


def strip_string(s: str) -> str:
    s = str(s).replace("\n", "").replace("\\!", "").replace("\\\\", "\\").replace("tfrac", "frac").replace("dfrac", "frac")
    s = s.replace("\\left", "").replace("\\right", "").replace("^{\\circ}", "").replace("^\\circ", "").replace("\\$", "")
    s = re.sub(r"\\text\{\s*([^}]*)\}", r"\1", s) if "\\text{ " in s else s
    s = s.replace("\\%", "").replace("%", "").replace(" .", " 0.").replace("{.", "{0.")
    if s.startswith("."):
        s = "0" + s
    if len(s.split("=")) == 2 and len(s.split("=")[0]) <= 2:
        s = s.split("=")[1]
    s = _fix_sqrt(s).replace(" ", "")
    s = _fix_fracs(s)
    if s == "0.5":
        s = "\\frac{1}{2}"
    m = re.fullmatch(r"(-?\d+)/(-?\d+)", s)
    if m:
        s = "\\frac{" + m.group(1) + "}{" + m.group(2) + "}"
    return s


def is_equiv(a, b) -> bool:
    if a is None or b is None:
        return a is None and b is None
    try:
        return strip_string(a) == strip_string(b)
    except Exception:
        return a == b


def compute_score(solution_str: str, ground_truth: str) -> float:
    try:
        boxed = last_boxed_only_string(solution_str)
        if boxed is not None and is_equiv(remove_boxed(boxed), ground_truth):
            return 1.0
    except Exception:
        pass
    return 0.0
