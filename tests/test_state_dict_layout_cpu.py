"""State-dict key names and shapes, pinned against lists written down from the reference's module definitions, so that
``model_weights.ckpt`` of a reference ``.nemo`` archive (``nemo/core/connectors/save_restore_connector.py:608-615``: a plain
``state_dict`` under that file name) loads key for key.

Sources of the expected names (reference tree):
* features: ``collections/asr/parts/preprocessing/features.py:319,336`` (buffers ``window``, ``fb`` under ``featurizer``);
* sub-sampling: ``parts/submodules/subsampling.py:184-257`` (``conv`` Sequential indices 0,2,3,5,6 and ``out``);
* Conformer layer: ``parts/submodules/conformer_modules.py`` (``norm_feed_forward1``, ``feed_forward1.linear1/2``, ``norm_self_att``,
  ``self_attn.{linear_q,linear_k,linear_v,linear_out,linear_pos,pos_bias_u,pos_bias_v}``, ``norm_conv``,
  ``conv.{pointwise_conv1,depthwise_conv,batch_norm,pointwise_conv2}``, ``norm_feed_forward2``, ``feed_forward2``, ``norm_out``);
* prediction network / joint: ``collections/asr/modules/rnnt.py`` (``prediction.embed``, ``prediction.dec_rnn.lstm`` from
  ``common/parts/rnn.py``, ``joint.pred``, ``joint.enc``, ``joint.joint_net``: activation, optional Dropout, Linear);
* Canary decoder: ``modules/transformer/transformer.py:190,199`` (``_embedding``, ``_decoder``), ``transformer_modules.py:93-100,
  174-177,238-239``, ``transformer_decoders.py:60-73,201``; head ``parts/submodules/token_classifier.py`` (``mlp.layer0``);
* speech-LLM backbone: Hugging Face Qwen3 parameter names (``model.layers.N.self_attn.{q,k,v,o}_proj``, ``q_norm``, ``k_norm``,
  ``mlp.{gate,up,down}_proj``, ``input_layernorm``, ``post_attention_layernorm``, ``model.norm``, ``lm_head``), which SALM loads
  unchanged (``collections/speechlm2/models/salm.py``).
"""
import torch


def _conformer_layer(prefix, d, ff, h, k):
    dk = d // h
    e = {}
    for n in ("norm_feed_forward1", "norm_self_att", "norm_conv", "norm_feed_forward2", "norm_out"):
        e[f"{prefix}.{n}.weight"] = (d,)
        e[f"{prefix}.{n}.bias"] = (d,)
    for n in ("feed_forward1", "feed_forward2"):
        e[f"{prefix}.{n}.linear1.weight"] = (ff, d)
        e[f"{prefix}.{n}.linear1.bias"] = (ff,)
        e[f"{prefix}.{n}.linear2.weight"] = (d, ff)
        e[f"{prefix}.{n}.linear2.bias"] = (d,)
    for n in ("linear_q", "linear_k", "linear_v", "linear_out"):
        e[f"{prefix}.self_attn.{n}.weight"] = (d, d)
        e[f"{prefix}.self_attn.{n}.bias"] = (d,)
    e[f"{prefix}.self_attn.linear_pos.weight"] = (d, d)
    e[f"{prefix}.self_attn.pos_bias_u"] = (h, dk)
    e[f"{prefix}.self_attn.pos_bias_v"] = (h, dk)
    e[f"{prefix}.conv.pointwise_conv1.weight"] = (2 * d, d, 1)
    e[f"{prefix}.conv.pointwise_conv1.bias"] = (2 * d,)
    e[f"{prefix}.conv.depthwise_conv.weight"] = (d, 1, k)
    e[f"{prefix}.conv.depthwise_conv.bias"] = (d,)
    for n, s in (("weight", (d,)), ("bias", (d,)), ("running_mean", (d,)), ("running_var", (d,)), ("num_batches_tracked", ())):
        e[f"{prefix}.conv.batch_norm.{n}"] = s
    e[f"{prefix}.conv.pointwise_conv2.weight"] = (d, d, 1)
    e[f"{prefix}.conv.pointwise_conv2.bias"] = (d,)
    return e


def _fastconformer_encoder(prefix, layers, d=1024, ff=4096, h=8, k=9, feat=80, ch=256):
    e = {f"{prefix}.pre_encode.out.weight": (d, ch * (feat // 8)), f"{prefix}.pre_encode.out.bias": (d,)}
    e[f"{prefix}.pre_encode.conv.0.weight"] = (ch, 1, 3, 3)
    e[f"{prefix}.pre_encode.conv.0.bias"] = (ch,)
    for dw, pw in ((2, 3), (5, 6)):
        e[f"{prefix}.pre_encode.conv.{dw}.weight"] = (ch, 1, 3, 3)
        e[f"{prefix}.pre_encode.conv.{dw}.bias"] = (ch,)
        e[f"{prefix}.pre_encode.conv.{pw}.weight"] = (ch, ch, 1, 1)
        e[f"{prefix}.pre_encode.conv.{pw}.bias"] = (ch,)
    for i in range(layers):
        e.update(_conformer_layer(f"{prefix}.layers.{i}", d, ff, h, k))
    return e


def test_tdt_06b_state_dict_matches_the_reference_layout():
    from speech_b200.models import EncDecRNNTBPEModel
    from speech_b200.models.configs import fastconformer_transducer_config

    L, V, D = 2, 1024, 5
    cfg = fastconformer_transducer_config("xlarge", vocab_size=V, loss="tdt", durations=(0, 1, 2, 3, 4), sigma=0.02, n_layers=L, sched=None)
    model = EncDecRNNTBPEModel(cfg)
    want = {"preprocessor.featurizer.window": (400,), "preprocessor.featurizer.fb": (1, 80, 257)}
    want.update(_fastconformer_encoder("encoder", L))
    want["decoder.prediction.embed.weight"] = (V + 1, 640)
    for layer in (0, 1):
        want[f"decoder.prediction.dec_rnn.lstm.weight_ih_l{layer}"] = (2560, 640)
        want[f"decoder.prediction.dec_rnn.lstm.weight_hh_l{layer}"] = (2560, 640)
        want[f"decoder.prediction.dec_rnn.lstm.bias_ih_l{layer}"] = (2560,)
        want[f"decoder.prediction.dec_rnn.lstm.bias_hh_l{layer}"] = (2560,)
    want.update({"joint.pred.weight": (640, 640), "joint.pred.bias": (640,), "joint.enc.weight": (640, 1024), "joint.enc.bias": (640,)})
    # joint_net = [activation, Linear] without dropout (index 1); the recipe's dropout 0.2 inserts a Dropout and moves it to 2
    want.update({"joint.joint_net.1.weight": (V + 1 + D, 640), "joint.joint_net.1.bias": (V + 1 + D,)})
    got = {k: tuple(v.shape) for k, v in model.state_dict().items()}
    assert got == want, (sorted(set(got) ^ set(want))[:10], [(k, got[k], want[k]) for k in got if k in want and got[k] != want[k]][:5])


def test_joint_dropout_moves_the_output_layer_to_index_two():
    from speech_b200.modules.rnnt import RNNTJoint

    j = RNNTJoint(jointnet={"encoder_hidden": 32, "pred_hidden": 16, "joint_hidden": 24, "activation": "relu", "dropout": 0.2},
                  num_classes=10, num_extra_outputs=5)
    assert "joint_net.2.weight" in j.state_dict() and tuple(j.state_dict()["joint_net.2.weight"].shape) == (16, 24)


def test_canary_decoder_and_head_match_the_reference_layout():
    from speech_b200.modules.transformer_nm import TokenClassifier, TransformerDecoderNM

    H, I, V, L = 1024, 4096, 16384, 2
    dec = TransformerDecoderNM(vocab_size=V, hidden_size=H, num_layers=L, inner_size=I, num_attention_heads=16, max_sequence_length=1024,
                               learn_positional_encodings=False, pre_ln=True, pre_ln_final_layer_norm=True)
    want = {"_embedding.token_embedding.weight": (V, H), "_embedding.position_embedding.pos_enc": (1024, H),
            "_embedding.token_type_embedding.weight": (2, H), "_embedding.layer_norm.weight": (H,), "_embedding.layer_norm.bias": (H,),
            "_decoder.final_layer_norm.weight": (H,), "_decoder.final_layer_norm.bias": (H,)}
    for i in range(L):
        p = f"_decoder.layers.{i}"
        for n in ("layer_norm_1", "layer_norm_2", "layer_norm_3"):
            want[f"{p}.{n}.weight"] = (H,)
            want[f"{p}.{n}.bias"] = (H,)
        for sub in ("first_sub_layer", "second_sub_layer"):
            for n in ("query_net", "key_net", "value_net", "out_projection"):
                want[f"{p}.{sub}.{n}.weight"] = (H, H)
                want[f"{p}.{sub}.{n}.bias"] = (H,)
        want[f"{p}.third_sub_layer.dense_in.weight"] = (I, H)
        want[f"{p}.third_sub_layer.dense_in.bias"] = (I,)
        want[f"{p}.third_sub_layer.dense_out.weight"] = (H, I)
        want[f"{p}.third_sub_layer.dense_out.bias"] = (H,)
    got = {k: tuple(v.shape) for k, v in dec.state_dict().items()}
    assert got == want, sorted(set(got) ^ set(want))[:10]
    head = TokenClassifier(hidden_size=H, num_classes=V, num_layers=1, log_softmax=True)
    assert {k: tuple(v.shape) for k, v in head.state_dict().items()} == {"mlp.layer0.weight": (V, H), "mlp.layer0.bias": (V,)}


def test_qwen3_backbone_uses_hugging_face_parameter_names():
    from speech_b200.speechlm.llm import CausalLM, LLMConfig

    cfg = LLMConfig(vocab_size=512, hidden_size=256, intermediate_size=768, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                    head_dim=128)
    m = CausalLM(cfg)
    want = {"model.embed_tokens.weight": (512, 256), "model.norm.weight": (256,), "lm_head.weight": (512, 256)}
    for i in range(2):
        p = f"model.layers.{i}"
        want.update({f"{p}.self_attn.q_proj.weight": (4 * 128, 256), f"{p}.self_attn.k_proj.weight": (2 * 128, 256),
                     f"{p}.self_attn.v_proj.weight": (2 * 128, 256), f"{p}.self_attn.o_proj.weight": (256, 4 * 128),
                     f"{p}.self_attn.q_norm.weight": (128,), f"{p}.self_attn.k_norm.weight": (128,),
                     f"{p}.mlp.gate_proj.weight": (768, 256), f"{p}.mlp.up_proj.weight": (768, 256), f"{p}.mlp.down_proj.weight": (256, 768),
                     f"{p}.input_layernorm.weight": (256,), f"{p}.post_attention_layernorm.weight": (256,)})
    got = {k: tuple(v.shape) for k, v in m.state_dict().items()}
    assert got == want, sorted(set(got) ^ set(want))[:10]
