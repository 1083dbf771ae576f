"""Model integrations under the reference's names: ``reskv.models.llama`` is the Hugging Face Llama
integration (``reskv_b200.models.hf_llama``), everything else comes from ``reskv_b200.models``."""


def __getattr__(name):
    import reskv_b200.models as models

    return getattr(models, name)
