/*
 * Binary layout of the two inputs of the render path: the immutable scene
 * blob (one per device) and the per-lane state records.  Plain C so that the
 * CUDA library, the CPU oracle and any foreign-function binding agree on it.
 *
 * Scene blob: `GD_HDR_WORDS` int32 words, then 128-byte aligned sections.  Word
 * GD_H_* holds a count; word GD_HDR_SECTION0 + GD_S_* holds the byte offset of
 * a section from the start of the blob.  The field meanings follow the
 * reference's device scene (src/gradoom/engine.py:607-1476, DeviceScenario).
 */
#ifndef GRADOOM_B200_LAYOUT_H
#define GRADOOM_B200_LAYOUT_H

#include <stdint.h>

#define GD_MAGIC 0x4744424C /* "GDBL" */
#define GD_VERSION 11
#define GD_HDR_WORDS 160
#define GD_HDR_SECTION0 48

/* view constants (src/gradoom/engine.py:1484-1487) */
#define GD_SCREEN_W 320
#define GD_VIEW_H 208
#define GD_SCREEN_H 240
#define GD_HUD_H 32
#define GD_OBS 84
#define GD_STACK 4

enum gd_header_word {
  GD_H_MAGIC = 0,
  GD_H_VERSION,
  GD_H_BYTES,        /* total blob size */
  GD_H_WALLS,        /* W */
  GD_H_SECTORS,      /* S */
  GD_H_VERTICES,     /* V distinct wall endpoints */
  GD_H_TEXTURES,     /* T */
  GD_H_TEX_H,        /* atlas slice height */
  GD_H_TEX_W,        /* atlas slice width */
  GD_H_SPRITES,      /* P */
  GD_H_SPR_H,
  GD_H_SPR_W,
  GD_H_WPN_PATCHES,  /* Q */
  GD_H_WPN_H,
  GD_H_WPN_W,
  GD_H_WPN_TICS,     /* last dim of the weapon frame tables */
  GD_H_STARTS,       /* player starts; the last one is the player */
  GD_H_DEATH_FRAMES,
  GD_H_XDEATH_FRAMES,
  GD_H_BLOCKING,     /* number of one-sided (blocking) walls */
  GD_H_NB_DIRECT,    /* 1 when every wall has <=1 same-pair neighbour per end */
  GD_H_WPN_AVAILABLE,
  GD_H_HUD_PATCHES,
  GD_H_UNSUPPORTED,  /* nonzero: scene uses a feature outside this path */
  GD_H_SEC_WALLS_N,  /* entries of GD_S_SEC_WALLS */
  GD_H_VTX_WALLS_N,  /* entries of GD_S_VTX_WALLS */
  GD_H_MASKED_WALLS_N, /* entries of GD_S_MASKED_WALLS */
  GD_H_FLOOR_GROUPS, /* distinct floor heights */
  GD_H_CEIL_GROUPS,  /* distinct ceiling heights */
  GD_H_ITEMS,        /* map items (pickups placed by the map) */
  GD_H_DECALS,       /* bullet-chip variants (0: the scene carries no decal bitmaps) */
  GD_H_DECAL_H,      /* atlas slice height */
  GD_H_DECAL_W,      /* atlas slice width = the width of every chip */
  GD_H_FRAGMENTS,    /* entries of GD_S_FRAG_FIXED: projection fragments of the lines a node builder split */
  GD_H_COUNT
};

enum gd_section {
  GD_S_WALLS = 0,     /* W x 4 f32   x1 y1 x2 y2 */
  GD_S_WALL_SECTORS,  /* W x 2 i32   front back(-1) */
  GD_S_WALL_LEN,      /* W f32       floor(hypot+0.5) */
  GD_S_SIDE_TEX,      /* W x 2 x 3 i32 (middle,bottom,top) */
  GD_S_SIDE_OFF,      /* W x 2 x 2 f32 */
  GD_S_WALL_VTX,      /* W x 2 i32   endpoint vertex ids */
  GD_S_VTX_OFF,       /* V+1 i32 CSR */
  GD_S_VTX_WALLS,     /* 2W i32 */
  GD_S_NB_DIRECT,     /* W x 4 i32: start idx, end idx (-1 none), start slot, end slot */
  GD_S_NB_OFF,        /* W+1 i32 CSR of same-sector-pair endpoint neighbours */
  GD_S_NB_IDX,        /* i32 */
  GD_S_NB_FLAGS,      /* i32 bit0 shares start, bit1 shares end */
  GD_S_SB_START_OFF,  /* W+1 solid-bridge CSR for the start endpoint */
  GD_S_SB_START_IDX,
  GD_S_SB_END_OFF,
  GD_S_SB_END_IDX,
  GD_S_SECTOR_F,      /* S x 2 f32 floor ceiling */
  GD_S_SECTOR_I,      /* S x 4 i32 light floor_tex ceil_tex closed(1: edges form closed loops) */
  GD_S_SEC_OFF,       /* S+1 CSR of incident walls (ascending) */
  GD_S_SEC_WALLS,
  GD_S_EDGE_OFF,      /* S+1 CSR of polygon edge walls (ascending) */
  GD_S_EDGE_WALLS,
  GD_S_BLOCKING,      /* B i32 wall index of each blocking segment */
  GD_S_TEX_INFO,      /* T x 4 i32 width height width_bits height_bits */
  GD_S_TEX_ATLAS,     /* T x H x W u8 */
  GD_S_PLAYPAL,       /* 256 x 3 u8 */
  GD_S_COLORMAP,      /* 34 x 256 u8 */
  GD_S_SPR_INFO,      /* P x 4 i32 width height left top */
  GD_S_SPR_ATLAS,     /* P x h x w u8 */
  GD_S_SPR_POST,      /* P x h x w u8: 255 transparent, else first row of the post */
  GD_S_ENEMY_WALK,    /* 6 x 4 x 8 i32 */
  GD_S_ENEMY_ATTACK,  /* 6 x 4 x 8 */
  GD_S_ENEMY_PAIN,    /* 6 x 8 */
  GD_S_DEATH_IDS,     /* 6 x F */
  GD_S_DEATH_COUNTS,  /* 6 */
  GD_S_DEATH_ENDS,    /* 6 x F cumulative frame ends */
  GD_S_XDEATH_IDS,
  GD_S_XDEATH_COUNTS,
  GD_S_XDEATH_ENDS,
  GD_S_PROJ_FLIGHT,   /* 3 x 2 x 8 */
  GD_S_PROJ_EXPL_IDS, /* 3 x 5 */
  GD_S_PROJ_EXPL_COUNTS, /* 3 */
  GD_S_PROJ_EXPL_ENDS,   /* 3 x 5 cumulative */
  GD_S_PROJ_EXPL_TOTAL,  /* 3 */
  GD_S_FOG_IDS,       /* 12 */
  GD_S_PUFF_IDS,      /* 4 */
  GD_S_STATIC_IDS,    /* 20 */
  GD_S_ADD_LUT,       /* 2 x 256 x 256 u8 [style][dst][src] */
  GD_S_TRANS_LUT,     /* 256 x 256 u8 [dst][src] */
  GD_S_WPN_INFO,      /* Q x 4 i32 width height left top */
  GD_S_WPN_ATLAS,     /* Q x h x w u8 */
  GD_S_WPN_OPAQUE,    /* Q x h x w u8 */
  GD_S_WPN_FRAME_IDS, /* 8 x 2 x tics i32 */
  GD_S_WPN_FLASH_IDS,
  GD_S_WPN_FLASH_LIGHTS,
  GD_S_HUD_INFO,      /* 70 x 4 i32 width height left top */
  GD_S_HUD_ATLAS,     /* 70 x 32 x 320 u8 */
  GD_S_HUD_OPAQUE,    /* 70 x 32 x 320 u8 */
  GD_S_FINESINE,      /* 8192 i32 */
  GD_S_FINETAN,       /* 4096 i32 */
  GD_S_STARTS,        /* starts x 4 f32: x y angle_rad floor_z */
  GD_S_RAY_OFFSETS,   /* 320 f32: -atan((col-160)/160), flat fallback rays */
  GD_S_RAY_COSCORR,   /* 320 f32: cos of the ray offsets */
  GD_S_TEX_ATLAS_COL, /* T x W x H u8: the atlas with every texture stored column-major */
  GD_S_SECTOR_BBOX,   /* S x 4 f32: xmin xmax ymin ymax over the sector's polygon edges */
  GD_S_MASKED_WALLS,  /* i32, ascending: two-sided walls with a middle texture on either side */
  GD_S_DAMAGE_ALPHA,  /* 114 f32: damage count -> red flash alpha (0..255), screen flashes */
  GD_S_FLOOR_GROUP_H,   /* distinct floor heights, descending (f32) */
  GD_S_FLOOR_GROUP_OFF, /* groups + 1 i32: CSR offsets into GD_S_FLOOR_GROUP_SEC */
  GD_S_FLOOR_GROUP_SEC, /* S i32: sectors of each floor height, ascending inside a group */
  GD_S_CEIL_GROUP_H,    /* distinct ceiling heights, ascending (f32) */
  GD_S_CEIL_GROUP_OFF,
  GD_S_CEIL_GROUP_SEC,
  GD_S_ITEM_POS,        /* items x 4 f32: x y z (floor of its sector + spawn height) 0 */
  GD_S_ITEM_INFO,       /* items x 2 i32: editor type id, sprite patch of its resting frame */
  GD_S_ITEM_ANIM,       /* 8 i32: bonus / armour animation frames (src/gradoom/engine.py:14258-14317) */
  GD_S_DECAL_INFO,      /* variants x 4 i32: height, left offset, top offset, 0 (src/gradoom/scenario.py:280-300) */
  GD_S_DECAL_ATLAS,     /* variants x h x w u8 grayscale chips, 0 = transparent */
  GD_S_DECAL_OPACITY,   /* 32 x 256 u8 [wall shade][chip texel] -> opacity 0..64 (src/gradoom/scenario.py:260-268) */
  GD_S_DECAL_BLACK,     /* 65 x 256 u8 [opacity][palette index] -> darkened palette index (scenario.py:269-272) */
  GD_S_WALL_FINE,       /* W x 2 i32: fine angle (0..8191) of the wall's direction seen from side 0 / side 1,
                           the tangent a chip on that side is laid out along (src/gradoom/engine.py:13818-13830) */
  GD_S_FRAG_OFF,        /* W+1 i32 CSR into GD_S_FRAG_FIXED; a line that was not split has an empty range */
  GD_S_FRAG_FIXED,      /* fragments x 4 i32: x1 y1 x2 y2 in 16.16, the pieces of a split line in the node
                           builder's order (src/gradoom/scenario.py:420-455, engine.py:745-767) */
  GD_S_COUNT
};

/*
 * Per-lane state record: 32 words (128 bytes).  The fields are the subset of
 * the reference engine's lane tensors the renderer reads
 * (src/gradoom/engine.py:1658-1739), narrowed to 32 bits.
 */
#define GD_LANE_WORDS 32
enum gd_lane_word {
  GD_L_X = 0,          /* f32 public x */
  GD_L_Y,              /* f32 public y */
  GD_L_ANGLE,          /* f32 public angle, radians */
  GD_L_VIEW_Z,         /* f32 */
  GD_L_X_FIXED,        /* i32 16.16 view x (public value if it was overridden) */
  GD_L_Y_FIXED,        /* i32 16.16 */
  GD_L_ANGLE_BAM,      /* u32 view angle BAM (public value if overridden) */
  GD_L_PITCH_BAM,      /* i32 */
  GD_L_FLAGS,          /* bit0 player dead, bit1 mugshot ouch, bit2 screen flashes on;
                          bits 8-15 damage count (0..113), bits 16-23 bonus count (0..255) */
  GD_L_EPISODE_TIME,   /* i32 */
  GD_L_BOB_FIXED,      /* i32 16.16 */
  GD_L_THINGS,         /* i32 number of thing records of this lane */
  GD_L_WEAPON,         /* i32 active weapon 0..7 */
  GD_L_WPN_COOLDOWN,   /* i32 weapon_state_cooldown */
  GD_L_WPN_FIRE_COUNT,
  GD_L_WPN_READY_TICS,
  GD_L_WPN_RAISE,
  GD_L_WPN_LOWER,
  GD_L_WPN_PENDING,    /* i32, <0 none */
  GD_L_HEALTH,         /* f32 */
  GD_L_ARMOR,          /* f32 */
  GD_L_READY_AMMO,     /* f32 cached hud_ready_ammo */
  GD_L_AMMO0,          /* f32 x4 hud_ammo_counts */
  GD_L_AMMO1,
  GD_L_AMMO2,
  GD_L_AMMO3,
  GD_L_WEAPONS_OWNED,  /* bit i = weapons[lane][i] != 0 */
  GD_L_FACE_INDEX,
  GD_L_PAIN_DIRECTION,
  GD_L_PAIN_TICS,
  GD_L_GRIN_TICS,
  GD_L_ATTACK_HELD
};

/*
 * Player kinematics record: 24 words (96 bytes) per lane, the state the per-tic
 * player movement reads and writes (src/gradoom/engine.py:1658-1744, narrowed to
 * 32 bits: every fixed-point value of a map fits).
 */
#define GD_PLAYER_WORDS 24
enum gd_player_word {
  GD_P_X_FIXED = 0,        /* i32 16.16 (_x_fixed) */
  GD_P_Y_FIXED,
  GD_P_MOMENTUM_X,         /* i32 16.16 (_momentum_x_fixed) */
  GD_P_MOMENTUM_Y,
  GD_P_ANGLE_BAM,          /* u32 (_angle_bam) */
  GD_P_PITCH_BAM,          /* i32 (_pitch_bam) */
  GD_P_BOB,                /* i32 16.16 (_player_bob_fixed) */
  GD_P_Z,                  /* f32 feet height */
  GD_P_VIEW_Z,             /* f32 camera height */
  GD_P_VIEW_HEIGHT,        /* f32 */
  GD_P_DELTA_VIEW_HEIGHT,  /* f32 */
  GD_P_VELOCITY_Z,         /* f32 */
  GD_P_FLOOR_Z,            /* f32 player_floor_z */
  GD_P_CEILING_Z,          /* f32 player_ceiling_z */
  GD_P_PREV_FLOOR_Z,       /* f32 previous_player_floor_z */
  GD_P_REACTION_TIME,      /* i32 tics of input freeze left */
  GD_P_TURN_HELD,          /* i32 turn_held_tics */
  GD_P_EPISODE_TIME,       /* i32 */
  GD_P_FLAGS,              /* GD_PLAYER_* */
  GD_P_RESERVED
};
#define GD_PLAYER_DEAD 1
#define GD_PLAYER_CHAINSAW_PULL 2

/*
 * Thing record: 16 bytes.  One per drawable actor of a lane, in the order the
 * reference concatenates them (src/gradoom/engine.py:14328-14682).
 */
typedef struct gd_thing {
  float x, y, z;
  uint16_t sprite;  /* index into the sprite patch tables */
  uint8_t flags;    /* bit0 alive, bit1 full-bright */
  int8_t style;     /* -1 normal, 0/1 additive LUT, -2 translucent LUT */
} gd_thing;

#define GD_THING_ALIVE 1
#define GD_THING_BRIGHT 2

/*
 * Decal record: 16 bytes.  One per slot of a lane's ring of bullet-chip decals
 * (src/gradoom/engine.py:1870-1884, written by 6257-6340).  A slot is in use when
 * serial >= 0; the chips of a lane are painted in ascending serial order.
 */
typedef struct gd_decal {
  int32_t serial;   /* hitscan_decal_serial, -1 = free slot */
  int16_t wall;     /* hitscan_decal_wall (clamped to the wall table when read) */
  uint16_t style;   /* hitscan_decal_style: variant + 5 * flip_x + 10 * flip_y + 20 * side */
  float along;      /* hitscan_decal_along: position of the impact on the wall, 0..1 */
  float z;          /* hitscan_decal_z: height of the impact */
} gd_decal;
#define GD_DECAL_SCALE 0.5f        /* map units per chip texel (src/gradoom/engine.py:133) */
#define GD_MAX_DECAL_SLOTS 1024    /* slots per lane the renderer accepts (src/gradoom/engine.py:132) */

#endif
