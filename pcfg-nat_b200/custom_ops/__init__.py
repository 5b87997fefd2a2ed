from .pcfg_loss import (cuda_pcfg_loss, cuda_pcfg_best_tree, cuda_pcfg_viterbi,  # noqa: F401
                        dag_logsoftmax_gather_inplace, viterbi_decoding, get_pcfg_kernel, proj_logsoftmax_gather)
