"""The SGLang attention-backend plugin surface, served by the B200 kernels.

Same entry point, hook table and call contracts as the reference's `lsa.sglang`
(`src/lsa/sglang/plugin.py`, `src/lsa/sglang/models/qwen3_5/backend.py`, `src/lsa/sglang/settings/design.py`):
`plugin.register` is what `[project.entry-points."sglang.srt.plugins"]` names; the settings arrive as the `"lsa"` block
of the model config; `backend.select_and_read` wraps `forward_extend` / `forward_decode`. SGLang itself is imported
only when a hook is registered, so everything else runs (and is tested) without it.
"""
