"""Switch a vllm-rlt installation over to the B200 handoff without editing its sources.

``install()`` rebinds the two names the reference resolves when it builds a stage worker's connector:
``vllm_rlt.pd.connector.PDStageConnector`` (used by tests and tools) and the ``PDStageConnector`` that
``vllm_rlt.pd.engine`` hands to its workers as ``connector_factory`` (vllm_rlt/pd/engine.py:24, :129).
Everything above the connector (coordinator, stage engine, scheduler, serving) is untouched.

Used as a pytest plugin (``-p vllm_rlt_b200.pd.dropin``) it installs itself before test modules are
imported, which is how this repository runs the reference's own connector tests against this
implementation.
"""

from __future__ import annotations


def install() -> None:
    import vllm_rlt.pd.connector as ref_connector

    from . import connector as mine

    ref_connector.PDStageConnector = mine.PDStageConnector
    ref_connector.RequestTransfer = mine.RequestTransfer
    try:
        import vllm_rlt.pd.engine as ref_engine
    except Exception:  # the coordinator needs optional serving dependencies; the connector swap does not
        ref_engine = None
    if ref_engine is not None:
        ref_engine.PDStageConnector = mine.PDStageConnector


def pytest_configure(config):  # pytest plugin hook
    install()
