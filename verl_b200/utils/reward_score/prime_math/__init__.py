"""Numina / PRIME math grading: take the final answer (last ``\\boxed{}``; else the text after "answer is"),
normalise both sides (LaTeX clean-up, units, thousands separators, ``\\frac``/``\\sqrt`` forms, percent), then
compare as strings, as numbers (relative 1e-6), as fractions, as tuples/intervals element-wise and, when
``sympy`` is importable, symbolically.

Parity target: ``verl/utils/reward_score/prime_math/{__init__ 411, grader 384, math_normalize 192}.py``;
``compute_score`` returns ``(is_correct, format_correct, extracted_answer)`` like the reference (:389-411).
"""

from __future__ import annotations

import re
from fractions import Fraction

from ..math_reward import last_boxed_only_string, remove_boxed, strip_string

__all__ = ["compute_score", "grade_answer", "normalize_final_answer", "match_answer"]

_UNIT_WORDS = ("degrees", "degree", "cm", "centimeters", "meters", "meter", "units", "unit", "square", "sq", "inches",
               "inch", "feet", "foot", "miles", "mph", "hours", "hour", "minutes", "seconds", "dollars", "cents", "percent")


def normalize_final_answer(ans: str) -> str:
    a = str(ans).strip()
    a = re.sub(r"\\text\{\s*([^}]*)\}", r"\1", a)
    a = re.sub(r"\\(?:mathrm|textbf|mathbf|boxed)\{([^}]*)\}", r"\1", a)
    a = a.replace("\\$", "").replace("$", "").replace("\\%", "%").replace("\\!", "").replace("\\,", "").replace("\\ ", " ")
    a = a.replace("\\left", "").replace("\\right", "").replace("dfrac", "frac").replace("tfrac", "frac")
    a = a.replace("^\\circ", "").replace("^{\\circ}", "").replace("°", "")
    a = re.sub(r"(?<=\d),(?=\d{3}\b)", "", a)  # 1,234 -> 1234
    for u in _UNIT_WORDS:
        a = re.sub(rf"(?<=[\d\s}}])\s*{u}\b\.?", "", a)
    a = a.strip().rstrip(".")
    if "=" in a and len(a.split("=")[0]) <= 3:  # "x = 5" -> "5"
        a = a.split("=")[-1]
    try:
        return strip_string(a)
    except Exception:
        return a.replace(" ", "")


def _to_number(s: str):
    t = s.replace(" ", "")
    pct = t.endswith("%")
    t = t[:-1] if pct else t
    m = re.fullmatch(r"(-?)\\frac\{(-?\d+)\}\{(-?\d+)\}", t)
    try:
        if m:
            v = Fraction(int(m.group(2)), int(m.group(3))) * (-1 if m.group(1) else 1)
        elif re.fullmatch(r"-?\d+/\d+", t):
            v = Fraction(t)
        else:
            v = Fraction(str(float(t))) if re.fullmatch(r"-?(\d+\.?\d*|\.\d+)([eE]-?\d+)?", t) else None
    except (ValueError, ZeroDivisionError):
        v = None
    if v is not None and pct:
        v = v / 100
    return v


def _split_top(s: str) -> list[str]:
    parts, depth, cur = [], 0, ""
    for ch in s:
        depth += ch in "({[" 
        depth -= ch in ")}]"
        if ch == "," and depth == 0:
            parts.append(cur)
            cur = ""
        else:
            cur += ch
    return parts + [cur]


def _sympy_equal(a: str, b: str) -> bool:
    try:
        import sympy
        from sympy.parsing.sympy_parser import parse_expr
    except Exception:
        return False
    try:
        conv = lambda s: re.sub(r"\\frac\{([^{}]*)\}\{([^{}]*)\}", r"((\1)/(\2))", s).replace("^", "**").replace("\\pi", "pi").replace("\\sqrt", "sqrt").replace("{", "(").replace("}", ")")
        return bool(sympy.simplify(parse_expr(conv(a)) - parse_expr(conv(b))) == 0)
    except Exception:
        return False


def grade_answer(given: str, truth: str) -> bool:
    if given is None:
        return False
    g, t = normalize_final_answer(given), normalize_final_answer(truth)
    if g == t:
        return True
    if not g or not t:
        return False
    ng, nt = _to_number(g), _to_number(t)
    if ng is not None and nt is not None:
        return abs(float(ng) - float(nt)) <= 1e-6 * max(1.0, abs(float(nt)))
    if g[0] in "([" and t[0] in "([" and g[-1] in ")]" and t[-1] in ")]":
        if (g[0], g[-1]) != (t[0], t[-1]):
            return False
        pg, pt = _split_top(g[1:-1]), _split_top(t[1:-1])
        return len(pg) == len(pt) and all(grade_answer(x, y) for x, y in zip(pg, pt))
    if (ng is None) != (nt is None):
        return _sympy_equal(g, t)
    return _sympy_equal(g, t)


def match_answer(response: str):
    """(format_ok, extracted answer). Boxed answers win; then "the answer is ..."; else the last line."""
    boxed = last_boxed_only_string(response)
    if boxed is not None:
        try:
            return True, remove_boxed(boxed)
        except Exception:
            pass
    m = re.findall(r"(?i)answer is[:\s]*([^\n]+)", response)
    if m:
        return True, m[-1].strip().rstrip(".").strip("$ ")
    lines = [l for l in response.strip().splitlines() if l.strip()]
    return False, (lines[-1].strip() if lines else "")


def compute_score(model_output: str, ground_truth: str):
    fmt, ans = match_answer(str(model_output))
    truth = str(ground_truth)
    if "\\boxed" in truth:
        truth = remove_boxed(last_boxed_only_string(truth))
    return grade_answer(ans, truth), fmt, ans
