"""A small re-implementation of the FileCheck directives the reference's EDSL tests use on the printed
program (plaidml/edsl/tests/edsl_test.cc): CHECK, CHECK-SAME, CHECK-NEXT and CHECK-DAG with `{{regex}}`
blocks and `[[name:regex]]` / `[[name]]` variables.  Horizontal whitespace is canonicalised on both
sides, as FileCheck does by default."""

import re

_TOKEN = re.compile(r"\{\{(.*?)\}\}|\[\[([A-Za-z_][A-Za-z0-9_]*)(?::(.*?))?\]\]")


class CheckFailure(AssertionError):
    pass


def _literal(text: str) -> str:
    parts = re.split(r"[ \t]+", text)
    return r"[ \t]+".join(re.escape(p) for p in parts)


def _compile(pattern: str, variables: dict):
    """The pattern as one regular expression; returns it and the variable names its groups define."""
    out, defined, pos = [], [], 0
    for m in _TOKEN.finditer(pattern):
        out.append(_literal(pattern[pos:m.start()]))
        pos = m.end()
        if m.group(1) is not None:
            out.append("(?:" + m.group(1) + ")")
        elif m.group(3) is not None:
            defined.append(m.group(2))
            out.append("(" + m.group(3) + ")")
        else:
            name = m.group(2)
            if name in defined:                      # defined earlier on the same line: a back-reference
                out.append("(?:\\%d)" % (defined.index(name) + 1))
            elif name in variables:
                out.append(re.escape(variables[name]))
            else:
                raise CheckFailure(f"undefined variable [[{name}]] in: {pattern}")
    out.append(_literal(pattern[pos:]))
    return re.compile("".join(out)), defined


def _canon(text: str) -> str:
    return "\n".join(re.sub(r"[ \t]+", " ", line).strip() for line in text.splitlines())


def run(directives, text: str) -> dict:
    """Applies [directive, pattern] pairs in order; raises CheckFailure naming the first that does not hold.
    Returns the variables captured on the way."""
    text = _canon(text)
    variables: dict = {}
    pos = 0                     # end of the last match
    i = 0
    while i < len(directives):
        kind, pattern = directives[i]
        pattern = pattern.strip()
        if kind == "CHECK-DAG":
            group_start, group_end = pos, pos
            while i < len(directives) and directives[i][0] == "CHECK-DAG":
                rx, names = _compile(directives[i][1].strip(), variables)
                m = rx.search(text, group_start)
                if not m:
                    raise CheckFailure(f"CHECK-DAG not found: {directives[i][1]}\n--- in:\n{text[group_start:]}")
                variables.update(zip(names, m.groups()))
                group_end = max(group_end, m.end())
                i += 1
            pos = group_end
            continue
        rx, names = _compile(pattern, variables)
        if kind == "CHECK":
            m = rx.search(text, pos)
        elif kind == "CHECK-SAME":
            eol = text.find("\n", pos)
            m = rx.search(text, pos, len(text) if eol < 0 else eol)
        elif kind == "CHECK-NEXT":
            eol = text.find("\n", pos)
            if eol < 0:
                m = None
            else:
                eol2 = text.find("\n", eol + 1)
                m = rx.search(text, eol + 1, len(text) if eol2 < 0 else eol2)
        else:
            raise CheckFailure(f"unsupported directive {kind}")
        if not m:
            raise CheckFailure(f"{kind} not found: {pattern}\n--- after offset {pos} of:\n{text}")
        variables.update(zip(names, m.groups()))
        pos = m.end()
        i += 1
    return variables
