{ neuralcuda.pas - Free Pascal binding of libcai_cuda.so, the B200 (sm_100a) decode backend.

  Place beside neural/neuralopencl.pas and build with -dCUDA. The unit has two parts:
    1. cdecl external declarations of include/cai_cuda.h (plain C types);
    2. TNeuralCudaBackend / TCudaDotProductKernel / TCudaDecodeSession, thin classes shaped like
       TEasyOpenCL / TDotProductSharedKernel / TNNetStreamingDecoder so that the call sites in
       neuralnetwork.pas (EnableOpenCL, ComputeOpenCL) and neuralchatengine.pas (LoadModel,
       GenerateFromIds) gain a CUDA twin with the same shape.

  This file cannot be compiled in the environment it was written in (no Free Pascal compiler there);
  it is kept deliberately thin. Errors follow the OpenCL unit's convention: integer status + message
  through ErrorProc, never an exception from the device layer. }
unit neuralcuda;

{$mode objfpc}{$H+}

interface

uses
  Classes, SysUtils, ctypes;

const
  CaiLib = 'cai_cuda';
  CAI_OK = 0; CAI_ERR_INVALID = 1; CAI_ERR_CUDA = 2; CAI_ERR_OOM = 3; CAI_ERR_STATE = 4; CAI_ERR_UNSUPPORTED = 5; CAI_ERR_COMM = 6;
  { resident storage types (ggml ids) }
  CAI_TYPE_F32 = 0; CAI_TYPE_F16 = 1; CAI_TYPE_Q4_0 = 2; CAI_TYPE_Q8_0 = 8;
  { load-time formats: decoded to fp32 on the device as they arrive }
  CAI_TYPE_Q4_1 = 3; CAI_TYPE_Q5_0 = 6; CAI_TYPE_Q5_1 = 7;
  CAI_TYPE_Q2_K = 10; CAI_TYPE_Q3_K = 11; CAI_TYPE_Q4_K = 12; CAI_TYPE_Q5_K = 13; CAI_TYPE_Q6_K = 14;
  CAI_TYPE_I8 = 24;      { KV cache: int8 codes + one fp32 scale per (head, position) row }
  CAI_TYPE_I8ROW = 124;  { the library's own int8 weights: K codes then the row's fp32 scale (TNNetVolume.QuantizeInt8) }
  CAI_ACT_NONE = 0; CAI_ACT_RELU = 1; CAI_ACT_SIGMOID = 2; CAI_ACT_TANH = 3;

type
  PCaiCtx = Pointer; PCaiLinear = Pointer; PCaiSdpa = Pointer; PCaiModel = Pointer; PCaiSession = Pointer; PCaiGguf = Pointer; PCaiMoeBank = Pointer;
  PPSingle = ^PSingle;

  TCaiLlamaConfig = record
    hidden, inter, layers, heads, kv_heads, head_dim, vocab: cint32;
    rms_eps, rope_theta: cfloat;
    tie_embeddings, qkv_bias, qk_norm, n_experts, top_k, norm_topk, moe_inter: cint32;
  end;

  TCaiSampling = record
    temperature: cfloat;
    top_k: cint32;
    top_p: cfloat;
    seed: cuint64;
  end;

{ Every entry point include/cai_cuda.h declares, in the header's order. }
function cai_cuda_init(device_id: cint; out out_ctx: PCaiCtx): cint; cdecl; external CaiLib;
function cai_cuda_shutdown(ctx: PCaiCtx): cint; cdecl; external CaiLib;
function cai_cuda_last_error(ctx: PCaiCtx; buf: PChar; buf_len: cint): cint; cdecl; external CaiLib;
function cai_cuda_device_info(ctx: PCaiCtx; sm_count: pcint; total_bytes: pcint64): cint; cdecl; external CaiLib;
function cai_cuda_launch_count(ctx: PCaiCtx; out_count: pcint64): cint; cdecl; external CaiLib;
function cai_cuda_is_checked_build(): cint; cdecl; external CaiLib;
function cai_cuda_set_wait_limit_us(ctx: PCaiCtx; limit_us: cuint): cint; cdecl; external CaiLib;
function cai_selftest_wait_timeout(ctx: PCaiCtx; which: cint; limit_us: cuint): cint; cdecl; external CaiLib;
function cai_dev_alloc(ctx: PCaiCtx; bytes: cint64; out out_dev: Pointer): cint; cdecl; external CaiLib;
function cai_dev_free(ctx: PCaiCtx; dev: Pointer): cint; cdecl; external CaiLib;
function cai_memcpy_h2d(ctx: PCaiCtx; dst_dev: Pointer; src_host: Pointer; bytes: cint64): cint; cdecl; external CaiLib;
function cai_memcpy_d2h(ctx: PCaiCtx; dst_host: Pointer; src_dev: Pointer; bytes: cint64): cint; cdecl; external CaiLib;
function cai_dev_sync(ctx: PCaiCtx): cint; cdecl; external CaiLib;
function cai_timer_begin(ctx: PCaiCtx): cint; cdecl; external CaiLib;
function cai_timer_end(ctx: PCaiCtx; out_ms: PSingle): cint; cdecl; external CaiLib;
function cai_flush_l2(ctx: PCaiCtx): cint; cdecl; external CaiLib;
function cai_dequantize(ctx: PCaiCtx; type_: cint; blocks_host: Pointer; rows: cint64; cols: cint64; out_host: PSingle): cint; cdecl; external CaiLib;
function cai_linear_create(ctx: PCaiCtx; type_: cint; blocks_host: Pointer; n_rows: cint64; k_cols: cint64; bias_host: PSingle; out out_: PCaiLinear): cint; cdecl; external CaiLib;
function cai_linear_create_int8(ctx: PCaiCtx; codes_host: pcint8; scales_host: PSingle; n_rows: cint64; k_cols: cint64; bias_host: PSingle; out out_: PCaiLinear): cint; cdecl; external CaiLib;
function cai_quantize_int8_rows(ctx: PCaiCtx; w_host: PSingle; rows: cint64; cols: cint64; codes_out_host: pcint8; scales_out_host: PSingle): cint; cdecl; external CaiLib;
function cai_linear_destroy(lin: PCaiLinear): cint; cdecl; external CaiLib;
function cai_linear_forward(lin: PCaiLinear; x_host: PSingle; batch: cint; y_host: PSingle; act: cint): cint; cdecl; external CaiLib;
function cai_linear_forward_dev(lin: PCaiLinear; x_dev: PSingle; batch: cint; y_dev: PSingle; act: cint): cint; cdecl; external CaiLib;
function cai_linear_forward_many(lins: PPointer; count: cint; x_dev: PSingle; batch: cint; y_dev: PSingle; iters: cint): cint; cdecl; external CaiLib;
function cai_linear_weight_bytes(lin: PCaiLinear; out_bytes: pcint64): cint; cdecl; external CaiLib;
function cai_linear_dequantize(lin: PCaiLinear; out_host: PSingle): cint; cdecl; external CaiLib;
function cai_linear_set_path(lin: PCaiLinear; path: cint): cint; cdecl; external CaiLib;
function cai_rmsnorm_dev(ctx: PCaiCtx; x_dev: PSingle; gain_dev: PSingle; y_dev: PSingle; tokens: cint; depth: cint; eps: cfloat): cint; cdecl; external CaiLib;
function cai_rope_dev(ctx: PCaiCtx; x_dev: PSingle; tokens: cint; depth: cint; head_dim: cint; position_offset: cint; theta_base: cfloat): cint; cdecl; external CaiLib;
function cai_swiglu_dev(ctx: PCaiCtx; x_dev: PSingle; y_dev: PSingle; tokens: cint; half_depth: cint): cint; cdecl; external CaiLib;
function cai_topk_gate_dev(ctx: PCaiCtx; router_logits_dev: PSingle; tokens: cint; n_experts: cint; top_k: cint; renorm: cint; expert_ids_dev: pcint32; gates_dev: PSingle): cint; cdecl; external CaiLib;
function cai_moe_bank_create(ctx: PCaiCtx; n_experts: cint; hidden: cint; expert_width: cint; type_: cint; out out_: PCaiMoeBank): cint; cdecl; external CaiLib;
function cai_moe_bank_destroy(b: PCaiMoeBank): cint; cdecl; external CaiLib;
function cai_moe_bank_upload(b: PCaiMoeBank; expert: cint; which: cint; blocks_host: Pointer): cint; cdecl; external CaiLib;
function cai_moe_bank_finalize(b: PCaiMoeBank): cint; cdecl; external CaiLib;
function cai_moe_gate_up_dev(b: PCaiMoeBank; x_dev: PSingle; slot_expert_dev: pcint32; tokens: cint; top_k: cint; hidden_out_dev: PSingle): cint; cdecl; external CaiLib;
function cai_moe_down_dev(b: PCaiMoeBank; hidden_dev: PSingle; slot_expert_dev: pcint32; slot_gate_dev: PSingle; tokens: cint; top_k: cint; out_dev: PSingle): cint; cdecl; external CaiLib;
function cai_sdpa_create(ctx: PCaiCtx; q_heads: cint; kv_heads: cint; head_dim: cint; max_ctx: cint; out out_: PCaiSdpa): cint; cdecl; external CaiLib;
function cai_sdpa_destroy(s: PCaiSdpa): cint; cdecl; external CaiLib;
function cai_sdpa_reset(s: PCaiSdpa): cint; cdecl; external CaiLib;
function cai_sdpa_truncate(s: PCaiSdpa; committed_len: cint): cint; cdecl; external CaiLib;
function cai_sdpa_cache_len(s: PCaiSdpa; out_len: pcint): cint; cdecl; external CaiLib;
function cai_sdpa_set_window(s: PCaiSdpa; window: cint): cint; cdecl; external CaiLib;
function cai_sdpa_enable_eviction(s: PCaiSdpa; sink_tokens: cint; recent_window: cint): cint; cdecl; external CaiLib;
function cai_sdpa_step_dev(s: PCaiSdpa; qkv_row_dev: PSingle; out_dev: PSingle): cint; cdecl; external CaiLib;
function cai_sdpa_step_noalloc(ctx: PCaiCtx; qkv_row_dev: PSingle; k_cache_dev: PSingle; v_cache_dev: PSingle; cache_len_dev: pcint32; q_heads: cint; kv_heads: cint; head_dim: cint; max_ctx: cint; out_dev: PSingle): cint; cdecl; external CaiLib;
function cai_model_create(ctx: PCaiCtx; const cfg: TCaiLlamaConfig; tp_rank: cint; tp_size: cint; out out_: PCaiModel): cint; cdecl; external CaiLib;
function cai_model_create_ep(ctx: PCaiCtx; const cfg: TCaiLlamaConfig; ep_rank: cint; ep_size: cint; out out_model: PCaiModel): cint; cdecl; external CaiLib;
function cai_model_destroy(m: PCaiModel): cint; cdecl; external CaiLib;
function cai_model_upload_tensor(m: PCaiModel; hf_name: PChar; type_: cint; data_host: Pointer; rows: cint64; cols: cint64; interleave_head_dim: cint): cint; cdecl; external CaiLib;
function cai_model_set_int8_weights(m: PCaiModel; on: cint): cint; cdecl; external CaiLib;
function cai_model_init_synthetic(m: PCaiModel; type_: cint; seed: cuint64; std: cfloat): cint; cdecl; external CaiLib;
function cai_model_read_tensor(m: PCaiModel; hf_name: PChar; out_host: Pointer; out_bytes_cap: cint64; out_type: pcint; out_rows: pcint64; out_cols: pcint64): cint; cdecl; external CaiLib;
function cai_gguf_open(path: PChar; out out_: PCaiGguf; err_buf: PChar; err_len: cint): cint; cdecl; external CaiLib;
function cai_gguf_close(g: PCaiGguf): cint; cdecl; external CaiLib;
function cai_gguf_last_error(g: PCaiGguf; buf: PChar; buf_len: cint): cint; cdecl; external CaiLib;
function cai_gguf_info(g: PCaiGguf; version: pcint; alignment: pcint; n_meta: pcint64; n_tensors: pcint64; data_start: pcint64): cint; cdecl; external CaiLib;
function cai_gguf_meta_key(g: PCaiGguf; index: cint64; key_buf: PChar; key_cap: cint; value_type: pcint): cint; cdecl; external CaiLib;
function cai_gguf_meta_int(g: PCaiGguf; key: PChar; out_: pcint64; found: pcint): cint; cdecl; external CaiLib;
function cai_gguf_meta_float(g: PCaiGguf; key: PChar; out_: pcdouble; found: pcint): cint; cdecl; external CaiLib;
function cai_gguf_meta_string(g: PCaiGguf; key: PChar; buf: PChar; cap: cint; found: pcint): cint; cdecl; external CaiLib;
function cai_gguf_meta_array_count(g: PCaiGguf; key: PChar; out_count: pcint64): cint; cdecl; external CaiLib;
function cai_gguf_tensor_info(g: PCaiGguf; index: cint64; name_buf: PChar; name_cap: cint; type_: pcint; ndims: pcint; shape8: pcint64; data_begin: pcint64; data_bytes: pcint64): cint; cdecl; external CaiLib;
function cai_gguf_find_tensor(g: PCaiGguf; name: PChar; out_index: pcint64): cint; cdecl; external CaiLib;
function cai_gguf_read_raw(g: PCaiGguf; index: cint64; out_host: Pointer; cap_bytes: cint64): cint; cdecl; external CaiLib;
function cai_gguf_decode(ctx: PCaiCtx; type_: cint; raw_host: Pointer; n_elems: cint64; out_host: PSingle): cint; cdecl; external CaiLib;
function cai_gguf_load_tensor(ctx: PCaiCtx; g: PCaiGguf; index: cint64; out_host: PSingle; cap_elems: cint64): cint; cdecl; external CaiLib;
function cai_gguf_llama_config(g: PCaiGguf; out cfg: TCaiLlamaConfig; max_positions: pcint64): cint; cdecl; external CaiLib;
function cai_model_load_gguf(ctx: PCaiCtx; path: PChar; tp_rank: cint; tp_size: cint; quantize_int8: cint; out out_model: PCaiModel; out out_cfg: TCaiLlamaConfig; out_max_positions: pcint64): cint; cdecl; external CaiLib;
function cai_model_finalize(m: PCaiModel): cint; cdecl; external CaiLib;
function cai_model_step_weight_bytes(m: PCaiModel; out_bytes: pcint64): cint; cdecl; external CaiLib;
function cai_session_create(m: PCaiModel; max_ctx: cint; batch: cint; kv_type: cint; out out_: PCaiSession): cint; cdecl; external CaiLib;
function cai_session_destroy(s: PCaiSession): cint; cdecl; external CaiLib;
function cai_session_reset(s: PCaiSession; seq: cint): cint; cdecl; external CaiLib;
function cai_session_truncate(s: PCaiSession; seq: cint; committed_len: cint): cint; cdecl; external CaiLib;
function cai_session_cache_len(s: PCaiSession; seq: cint; out_len: pcint): cint; cdecl; external CaiLib;
function cai_session_enable_eviction(s: PCaiSession; sink_tokens: cint; recent_window: cint): cint; cdecl; external CaiLib;
function cai_session_set_window(s: PCaiSession; window: cint): cint; cdecl; external CaiLib;
function cai_session_fill_for_benchmark(s: PCaiSession; n_rows: cint): cint; cdecl; external CaiLib;
function cai_session_step(s: PCaiSession; tokens_host: pcint32; abs_pos_host: pcint32; logits_out_host: PSingle; argmax_out_host: pcint32): cint; cdecl; external CaiLib;
function cai_session_decode_greedy(s: PCaiSession; tokens_host: pcint32; n_steps: cint; out_tokens_host: pcint32): cint; cdecl; external CaiLib;
function cai_session_step_topk(s: PCaiSession; tokens_host: pcint32; abs_pos_host: pcint32; k: cint; temperature: cfloat; ids_out_host: pcint32; probs_out_host: PSingle): cint; cdecl; external CaiLib;
function cai_session_decode_sampled(s: PCaiSession; tokens_host: pcint32; n_steps: cint; const opt: TCaiSampling; uniforms_host: PSingle; out_tokens_host: pcint32): cint; cdecl; external CaiLib;
function cai_sampling_uniform(seed: cuint64; step: cuint64; seq: cuint64; out_u: PSingle): cint; cdecl; external CaiLib;
function cai_session_prefill(s: PCaiSession; tokens_host: pcint32; n_tokens: cint): cint; cdecl; external CaiLib;
function cai_session_profile(s: PCaiSession; tokens_host: pcint32; n_steps: cint; out_ms: PSingle; out_launches: pcint64): cint; cdecl; external CaiLib;
function cai_session_snapshot(s: PCaiSession): cint; cdecl; external CaiLib;
function cai_session_restore(s: PCaiSession): cint; cdecl; external CaiLib;
function cai_session_logits_dev(s: PCaiSession; out_dev: PPSingle): cint; cdecl; external CaiLib;
function cai_session_read_kv_row(s: PCaiSession; layer: cint; seq: cint; kv_head: cint; pos: cint; k_out_host: PSingle; v_out_host: PSingle; k_codes_host: pcint8; v_codes_host: pcint8; scales_host: PSingle): cint; cdecl; external CaiLib;
function cai_session_uses_step_kernel(s: PCaiSession; out_flag: pcint): cint; cdecl; external CaiLib;
function cai_session_step_trace(s: PCaiSession; tokens_host: pcint32; out_ns: pcint64; out_family: pcint32; cap: cint; out_n: pcint): cint; cdecl; external CaiLib;
function cai_session_last_kv_bytes(s: PCaiSession; out_bytes: pcint64): cint; cdecl; external CaiLib;
function cai_comm_unique_id(out_id: PByte): cint; cdecl; external CaiLib;
function cai_comm_init(ctx: PCaiCtx; rank: cint; world: cint; id: PByte): cint; cdecl; external CaiLib;
function cai_comm_allreduce_dev(ctx: PCaiCtx; buf_dev: PSingle; count: cint64): cint; cdecl; external CaiLib;

type
  TCudaErrorProc = procedure(const Msg: string) of object;

  { Context owner: the CUDA twin of TEasyOpenCL. }
  TNeuralCudaBackend = class
  private
    FCtx: PCaiCtx;
    FErrorProc: TCudaErrorProc;
  public
    constructor Create(DeviceId: integer);
    destructor Destroy; override;
    function Check(Status: cint): boolean;        // false + ErrorProc(message) on failure
    property Ctx: PCaiCtx read FCtx;
    property ErrorProc: TCudaErrorProc read FErrorProc write FErrorProc;
  end;

  { Resident quantized linear layer: the CUDA twin of TDotProductSharedKernel's int8 mode. }
  TCudaDotProductKernel = class
  private
    FBackend: TNeuralCudaBackend;
    FLin: PCaiLinear;
    FNumAs, FSize: integer;
  public
    constructor Create(Backend: TNeuralCudaBackend);
    destructor Destroy; override;
    function PrepareForComputeQuant(GGMLType: integer; Blocks: Pointer; NumAs, pSize: integer; Bias: PSingle): integer;
    procedure ComputeQuant(X: PSingle; NumBs: integer; Y: PSingle; pActFN: integer);
    function PrepareForComputeInt8(Codes: pcint8; Scales: PSingle; NumAs, pSize: integer; Bias: PSingle): integer;
    function QuantReady: boolean;
  end;

  { Whole-model decode session: the CUDA twin of TNNetStreamingDecoder for a CUDA-capable net. }
  TCudaDecodeSession = class
  private
    FBackend: TNeuralCudaBackend;
    FModel: PCaiModel;
    FSession: PCaiSession;
    FVocab: integer;
    FMaxPositions: int64;
  public
    constructor Create(Backend: TNeuralCudaBackend; const Cfg: TCaiLlamaConfig);
    { BuildFromGGUFEx on the C side: parse, decode and upload the whole file; the model arrives finalized. }
    constructor CreateFromGGUF(Backend: TNeuralCudaBackend; const FileName: string; pQuantizeInt8: boolean);
    destructor Destroy; override;
    procedure SetInt8Weights(pOn: boolean);                  // the importer's pQuantizeInt8; call before UploadTensor
    procedure UploadTensor(const HFName: string; GGMLType: integer; Data: Pointer; Rows, Cols: int64; InterleaveHeadDim: integer);
    procedure Open(MaxContext: integer);                     // finalize + create the session
    procedure Reset;
    procedure TruncateTo(CommittedLen: integer);
    function StepForward(Token, AbsPos: integer; Logits: PSingle): integer;   // returns the argmax
  end;

implementation

constructor TNeuralCudaBackend.Create(DeviceId: integer);
begin
  inherited Create;
  if cai_cuda_init(DeviceId, FCtx) <> CAI_OK then FCtx := nil;
end;

destructor TNeuralCudaBackend.Destroy;
begin
  if FCtx <> nil then cai_cuda_shutdown(FCtx);
  inherited Destroy;
end;

function TNeuralCudaBackend.Check(Status: cint): boolean;
var
  Buf: array[0..1023] of char;
begin
  Result := Status = CAI_OK;
  if (not Result) and Assigned(FErrorProc) then
  begin
    cai_cuda_last_error(FCtx, @Buf[0], Length(Buf));
    FErrorProc('CUDA backend error ' + IntToStr(Status) + ': ' + StrPas(@Buf[0]));
  end;
end;

constructor TCudaDotProductKernel.Create(Backend: TNeuralCudaBackend);
begin
  inherited Create;
  FBackend := Backend;
end;

destructor TCudaDotProductKernel.Destroy;
begin
  if FLin <> nil then cai_linear_destroy(FLin);
  inherited Destroy;
end;

function TCudaDotProductKernel.PrepareForComputeQuant(GGMLType: integer; Blocks: Pointer; NumAs, pSize: integer; Bias: PSingle): integer;
begin
  if FLin <> nil then begin cai_linear_destroy(FLin); FLin := nil; end;
  FNumAs := NumAs; FSize := pSize;
  Result := cai_linear_create(FBackend.Ctx, GGMLType, Blocks, NumAs, pSize, Bias, FLin);
  FBackend.Check(Result);
end;

function TCudaDotProductKernel.PrepareForComputeInt8(Codes: pcint8; Scales: PSingle; NumAs, pSize: integer; Bias: PSingle): integer;
begin
  if FLin <> nil then begin cai_linear_destroy(FLin); FLin := nil; end;
  FNumAs := NumAs; FSize := pSize;
  Result := cai_linear_create_int8(FBackend.Ctx, Codes, Scales, NumAs, pSize, Bias, FLin);
  FBackend.Check(Result);
end;

function TCudaDotProductKernel.QuantReady: boolean;
begin
  Result := FLin <> nil;
end;

procedure TCudaDotProductKernel.ComputeQuant(X: PSingle; NumBs: integer; Y: PSingle; pActFN: integer);
begin
  FBackend.Check(cai_linear_forward(FLin, X, NumBs, Y, pActFN));
end;

constructor TCudaDecodeSession.Create(Backend: TNeuralCudaBackend; const Cfg: TCaiLlamaConfig);
begin
  inherited Create;
  FBackend := Backend;
  FVocab := Cfg.vocab;
  FBackend.Check(cai_model_create(Backend.Ctx, Cfg, 0, 1, FModel));
end;

constructor TCudaDecodeSession.CreateFromGGUF(Backend: TNeuralCudaBackend; const FileName: string; pQuantizeInt8: boolean);
var
  Cfg: TCaiLlamaConfig;
begin
  inherited Create;
  FBackend := Backend;
  if FBackend.Check(cai_model_load_gguf(Backend.Ctx, PChar(FileName), 0, 1, Ord(pQuantizeInt8), FModel, Cfg, @FMaxPositions)) then
    FVocab := Cfg.vocab;
end;

procedure TCudaDecodeSession.SetInt8Weights(pOn: boolean);
begin
  FBackend.Check(cai_model_set_int8_weights(FModel, Ord(pOn)));
end;

destructor TCudaDecodeSession.Destroy;
begin
  if FSession <> nil then cai_session_destroy(FSession);
  if FModel <> nil then cai_model_destroy(FModel);
  inherited Destroy;
end;

procedure TCudaDecodeSession.UploadTensor(const HFName: string; GGMLType: integer; Data: Pointer; Rows, Cols: int64; InterleaveHeadDim: integer);
begin
  FBackend.Check(cai_model_upload_tensor(FModel, PChar(HFName), GGMLType, Data, Rows, Cols, InterleaveHeadDim));
end;

procedure TCudaDecodeSession.Open(MaxContext: integer);
begin
  if FBackend.Check(cai_model_finalize(FModel)) then
    FBackend.Check(cai_session_create(FModel, MaxContext, 1, CAI_TYPE_F32, FSession));
end;

procedure TCudaDecodeSession.Reset;
begin
  FBackend.Check(cai_session_reset(FSession, -1));
end;

procedure TCudaDecodeSession.TruncateTo(CommittedLen: integer);
begin
  FBackend.Check(cai_session_truncate(FSession, 0, CommittedLen));
end;

function TCudaDecodeSession.StepForward(Token, AbsPos: integer; Logits: PSingle): integer;
var
  Tok, Pos, Arg: cint32;
begin
  Tok := Token; Pos := AbsPos; Arg := 0;
  FBackend.Check(cai_session_step(FSession, @Tok, @Pos, Logits, @Arg));
  Result := Arg;
end;

end.
