"""tidaldecode_b200 — TidalDecode's decode-time attention path on B200 (sm_100a).

Importing the package does not load the CUDA library; the submodules that run kernels
(`ops`, `_kernels`, `utils`, `attention`, `llama`, `enable_tidal`, `sharded`) do, and raise if
`libtidal_b200.so` has not been built (`python -m tidaldecode_b200.build`).

    from tidaldecode_b200.llama import LlamaForCausalLM, LlamaConfig      # kernel-path model (tidal.LlamaForCausalLM)
    from tidaldecode_b200.enable_tidal import enable_tidal                # PyTorch-path switch (src.enable_tidal)
    import tidaldecode_b200.utils as tidal_utils                          # operator façade (tidal.utils)
    import tidaldecode_b200._kernels as _kernels                          # extension drop-in (tidal._kernels)
"""

__version__ = "0.1.0"
