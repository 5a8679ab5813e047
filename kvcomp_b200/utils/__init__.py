"""Host-side helpers the reference keeps in utils/: quant modes, block cutting, RoPE, the config object."""
