"""The code blocks of the user guide run (CPU), chapter by chapter, sharing one namespace."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_guide_snippets_run():
    text = open(os.path.join(ROOT, "docs", "GUIDE.md")).read()
    blocks = re.findall(r"```python\n(.*?)```", text, flags=re.S)
    assert len(blocks) >= 7
    from gonn_b200.tensor import api
    registry = dict(api._REGISTRY)            # the "extending" chapter registers a demo op
    ns = {}
    try:
        for code in blocks:
            if "init_process_group" in code:  # the multi-process chapter needs a launcher
                continue
            exec(compile(code, "<guide>", "exec"), ns)
    finally:
        api._REGISTRY.clear()
        api._REGISTRY.update(registry)
